"""tcgen05 GEMM kernel against an fp32 PyTorch reference of the same contraction."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn, bias):
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    out = af @ bf
    if bias is not None:
        out = out + bias
    return out


def _check(out, ref, k):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 if out.dtype == torch.bfloat16 else 2e-3
    assert err / scale < tol, f"relative error {err / scale:.3e} (K={k})"


@pytest.mark.parametrize(
    "m,n,k",
    [(128, 256, 64), (256, 512, 256), (384, 256, 1024), (200, 136, 72), (1024, 1024, 2048), (129, 72, 200)],
)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_matches_fp32(m, n, k, a_mn, b_mn):
    from stacr_b200.ops import _lib
    from stacr_b200.ops.gemm import gemm

    if (a_mn and m % 8) or (b_mn and n % 8) or ((not a_mn or not b_mn) and k % 8):
        pytest.skip("leading dimension must be a multiple of 8 elements")
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n * 3 + k)
    a = torch.randn((k, m) if a_mn else (m, k), device="cuda", generator=g).bfloat16()
    b = torch.randn((k, n) if b_mn else (n, k), device="cuda", generator=g).bfloat16()
    bias = torch.randn(n, device="cuda", generator=g)
    ref = _ref(a, b, a_mn, b_mn, bias)
    for dtype in (torch.bfloat16, torch.float32):
        out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, out_dtype=dtype)
        torch.cuda.synchronize()
        _lib.check_status()
        _check(out, ref, k)


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("a_mn", [False, True])
def test_gemm_tile_widths_and_split_k(bn, a_mn):
    from stacr_b200.ops import _lib
    from stacr_b200.ops.gemm import gemm

    m, n, k = 512, bn, 4096
    g = torch.Generator(device="cuda").manual_seed(bn)
    a = torch.randn((k, m) if a_mn else (m, k), device="cuda", generator=g).bfloat16()
    b = torch.randn(n, k, device="cuda", generator=g).bfloat16()
    ref = _ref(a, b, a_mn, False, None)
    out = gemm(a, b, a_mn=a_mn, bn=bn, out_dtype=torch.float32)
    out_split = gemm(a, b, a_mn=a_mn, bn=bn, splits=8)
    torch.cuda.synchronize()
    _lib.check_status()
    _check(out, ref, k)
    _check(out_split, ref, k)


def test_gemm_repeatable_bits():
    from stacr_b200.ops.gemm import gemm

    a = torch.randn(1024, 512, device="cuda").bfloat16()
    b = torch.randn(768, 512, device="cuda").bfloat16()
    first = gemm(a, b)
    for _ in range(3):
        assert torch.equal(first, gemm(a, b))


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k,out_dtype", [(512, 512, 256, torch.bfloat16), (1024, 768, 192, torch.float32), (704, 520, 136, torch.bfloat16)])
def test_cta_pair_kernel_matches_fp32_reference(a_mn, b_mn, m, n, k, out_dtype):
    """tcgen05.mma.cta_group::2 on 256 x 256 pair tiles, all operand layouts, ragged edges and a bias."""
    from stacr_b200.ops import _lib
    from stacr_b200.ops.gemm import gemm

    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    bias = torch.randn(n, device="cuda")
    ref = a.float() @ b.float().t() + bias
    aa = a.t().contiguous() if a_mn else a
    bb = b.t().contiguous() if b_mn else b
    got = gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, bias=bias, out_dtype=out_dtype, two_cta=True)
    _lib.check_status()
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    assert float((got.float() - ref).abs().max() / ref.abs().max()) < tol


@pytest.mark.parametrize("m,n,k", [(129, 72, 200), (257, 264, 136), (1000, 520, 328)])
@pytest.mark.parametrize("two_cta", [False, True])
def test_ragged_edge_tiles_elementwise(m, n, k, two_cta):
    """Shapes that are no multiple of any tile: every element of the last partial row and column tiles is checked against
    the fp32 product of the same bf16 operands (integers, so the fp32 result is exact and the comparison is elementwise)."""
    from stacr_b200.ops import _lib
    from stacr_b200.ops.gemm import gemm

    if two_cta and (m < 512 or n < 512):
        pytest.skip("the CTA-pair kernel takes shapes of at least 512 x 512")
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randint(-3, 4, (m, k), device="cuda", generator=g).bfloat16()
    b = torch.randint(-3, 4, (n, k), device="cuda", generator=g).bfloat16()
    ref = a.float() @ b.float().t()
    out = gemm(a, b, out_dtype=torch.float32, two_cta=two_cta, bn=256 if two_cta else None)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(out, ref)
    edge_rows, edge_cols = m - m % 128, n - n % 128
    assert torch.equal(out[edge_rows:], ref[edge_rows:]) and torch.equal(out[:, edge_cols:], ref[:, edge_cols:])
