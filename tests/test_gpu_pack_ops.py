"""Index-stream encodings, per-tensor codecs, row moves and the fixed-threshold pass against plain PyTorch references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _random_flat(rows, n, nnz, seed, dtype=torch.int32):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randperm(rows * n, device="cuda", generator=g)[:nnz].to(dtype)


@pytest.mark.parametrize("rows,n,nnz,dtype", [(64, 100, 500, torch.int32), (2048, 8192, 83886, torch.int32), (300, 40000, 20000, torch.int64), (5, 7, 35, torch.int32)])
@pytest.mark.parametrize("mode", ["csr", "delta"])
def test_device_index_encodings_round_trip_and_match_the_framework_encoding(rows, n, nnz, dtype, mode):
    from stacr_b200.index_compression import compress_indices, decompress_indices

    flat = _random_flat(rows, n, nnz, seed=rows + nnz, dtype=dtype)
    packed = compress_indices(flat, rows, n, mode)
    assert packed.col_indices.is_cuda and packed.nnz == nnz
    back = decompress_indices(packed)
    assert back.dtype == dtype and torch.equal(back, flat)                       # original order restored
    unordered = decompress_indices(packed, restore_order=False).long()
    ref = compress_indices(flat.cpu(), rows, n, mode)                             # framework path on the host
    if mode == "csr":
        assert torch.equal(packed.row_ptrs.cpu().long(), ref.row_ptrs.long())
        assert packed.col_indices.dtype == ref.col_indices.dtype
        # the same entries in every row (order inside a row is free)
        assert torch.equal(unordered.sort().values.cpu(), flat.long().sort().values.cpu())
        rows_of = unordered // n
        assert bool((rows_of[1:] >= rows_of[:-1]).all())
    else:
        assert torch.equal(unordered.cpu(), flat.long().sort().values.cpu())
        assert packed.col_indices.dtype == ref.col_indices.dtype and torch.equal(packed.col_indices.cpu(), ref.col_indices)
        assert int(packed.delta_base) == int(ref.delta_base)
    assert packed.memory_bytes() == ref.memory_bytes()


def test_delta_encoding_with_a_row_too_long_for_the_in_row_sorter_falls_back():
    from stacr_b200.index_compression import compress_indices, decompress_indices

    rows, n = 4, 8192
    flat = torch.cat((torch.arange(5000, device="cuda", dtype=torch.int32).flip(0), torch.tensor([3 * n + 5, 2 * n + 1], device="cuda", dtype=torch.int32)))
    packed = compress_indices(flat, rows, n, "delta")
    assert torch.equal(decompress_indices(packed), flat)


def test_out_of_range_index_is_reported():
    from stacr_b200.ops import pack_ops

    flat = torch.tensor([0, 5, 64 * 100], device="cuda", dtype=torch.int32)
    with pytest.raises(ValueError):
        pack_ops.csr_pack(flat, 64, 100, narrow_cols=True, want_order=False, want_inverse=True)


@pytest.mark.parametrize("shape,dtype", [((8192, 8), torch.bfloat16), ((4097, 32), torch.bfloat16), ((1001,), torch.float32), ((3,), torch.bfloat16)])
@pytest.mark.parametrize("bits", [8, 4])
def test_symmetric_codecs_match_the_framework_codecs(shape, dtype, bits):
    from stacr_b200 import adaptive
    from stacr_b200.ops import pack_ops

    g = torch.Generator(device="cuda").manual_seed(3)
    x = (2.5 * torch.randn(*shape, device="cuda", generator=g)).to(dtype)
    codes, scale = pack_ops.quantize_symmetric(x, bits)
    xf = x.float().cpu()
    if bits == 8:
        want_q, want_s = adaptive.quantize_int8(xf)
        assert torch.equal(codes.cpu(), want_q) and codes.shape == x.shape
    else:
        want_q, want_s, length = adaptive.quantize_int4(xf)
        assert length == x.numel() and torch.equal(codes.cpu(), want_q)
        torch.testing.assert_close(adaptive.dequantize_int4(codes, scale, x.numel()).cpu(), adaptive.dequantize_int4(want_q, want_s, length))
    torch.testing.assert_close(scale.cpu(), want_s.float(), rtol=1e-6, atol=0)
    torch.testing.assert_close(pack_ops.sum_squares(x.contiguous()).cpu(), xf.square().sum(), rtol=1e-4, atol=1e-6)
    zeros = torch.zeros(16, device="cuda", dtype=dtype)
    zc, zs = pack_ops.quantize_symmetric(zeros, bits)
    assert float(zs) == 1.0 and int(zc.to(torch.int32).sum()) == (0 if bits == 8 else 8 * 0x88)


def test_row_gather_and_scatter():
    from stacr_b200.ops import pack_ops

    g = torch.Generator(device="cuda").manual_seed(5)
    src = torch.randn(300, 768, device="cuda", generator=g).bfloat16()
    index = torch.randperm(300, device="cuda", generator=g)[:123]
    got = pack_ops.move_rows(src, index)
    assert torch.equal(got, src[index])
    dst = torch.zeros(300, 768, device="cuda", dtype=torch.bfloat16)
    pack_ops.move_rows(got, index, scatter_into=dst)
    want = torch.zeros_like(dst)
    want[index] = got
    assert torch.equal(dst, want)


@pytest.mark.parametrize("rows,n,r", [(1024, 2048, 8), (700, 1280, 16), (128, 64, 32)])
def test_fixed_threshold_pass_lists_exactly_the_entries_above_the_threshold(rows, n, r):
    from stacr_b200.ops import _lib, stacr_ops

    g = torch.Generator(device="cuda").manual_seed(9)
    low = torch.randn(rows, r, device="cuda", generator=g) @ torch.randn(r, n, device="cuda", generator=g)
    x = (low + 0.3 * torch.randn(rows, n, device="cuda", generator=g)).bfloat16()
    qb = torch.linalg.qr(torch.randn(n, r, device="cuda", generator=g)).Q.bfloat16().contiguous()
    c = (x.float() @ qb.float()).bfloat16().contiguous()
    acc = torch.zeros(rows, n, device="cuda")
    for j in range(r):
        acc = (c[:, j:j + 1].double() * qb[:, j].double()[None, :] + acc.double()).float()
    e = (x.float() - acc).bfloat16().reshape(-1)
    thr = float(e.float().abs().quantile(0.99).item()) if e.numel() < 2 ** 24 else 0.8
    for _ in range(2):                                  # the second call reuses the remembered capacity
        idx, val = stacr_ops.residual_above(x, c, qb, thr)
        torch.cuda.synchronize()
        _lib.check_status()
        want = (e.float().abs() > thr).nonzero(as_tuple=True)[0]
        got = idx.sort().values
        both = len(set(got.tolist()) ^ set(want.tolist()))
        assert both <= 2, (both, got.numel(), want.numel())     # tensor-core vs chained-FMA rounding at the threshold itself
        assert (val.float().abs() > thr).all()


def test_mask_aware_row_moves_are_differentiable_and_match_index_ops():
    from stacr_b200.protocols.attention import gather_rows, scatter_rows

    g = torch.Generator(device="cuda").manual_seed(11)
    flat = torch.randn(200, 256, device="cuda", generator=g).bfloat16().requires_grad_(True)
    rows = torch.randperm(200, device="cuda", generator=g)[:77].sort().values
    picked = gather_rows(flat, rows)
    out = scatter_rows(picked * 2, rows, 200)
    ref_in = flat.detach().clone().requires_grad_(True)
    ref = torch.zeros(200, 256, device="cuda", dtype=torch.bfloat16).index_copy(0, rows, ref_in.index_select(0, rows) * 2)
    assert torch.equal(out, ref)
    w = torch.randn(200, 256, device="cuda", generator=g).bfloat16()
    (out * w).sum().backward()
    (ref * w).sum().backward()
    assert torch.equal(flat.grad, ref_in.grad)


def test_per_row_int8_codec_and_boundary_codec_on_kernels():
    from stacr_b200.ops import pack_ops
    from stacr_b200.protocols.checkpointing import CheckpointBoundaryCodec, STACRCheckpointSpec

    g = torch.Generator(device="cuda").manual_seed(13)
    coeff = torch.randn(1000, 16, device="cuda", generator=g) * torch.linspace(0.01, 30.0, 1000, device="cuda")[:, None]
    q, scale = pack_ops.quantize_rows_int8(coeff)
    want_scale = (coeff.abs().amax(1, keepdim=True) / 127.0).clamp_min(torch.finfo(torch.float32).tiny)
    torch.testing.assert_close(scale, want_scale, rtol=1e-6, atol=0)
    want_q = torch.round(coeff / want_scale).clamp_(-127, 127).to(torch.int8)
    diff = (q.int() - want_q.int()).abs()
    # the kernel multiplies by the reciprocal of the scale: a value that lands within an ulp of a half-integer may round the other way
    assert int(diff.max()) <= 1 and float((diff > 0).float().mean()) < 1e-3
    deq = pack_ops.dequantize_rows_int8(q, scale)
    torch.testing.assert_close(deq.float(), (q.float() * scale).bfloat16().float(), rtol=0, atol=0)
    # the boundary codec end to end on a bf16 tensor with low-rank structure: small reconstruction error, int8 payload
    hidden, rank = 512, 16
    spec = STACRCheckpointSpec(site_id="blk0", module_type="block", model_family="gpt2", hidden_size=hidden, rank=rank, basis_dtype=torch.float32,
                               min_numel=1, warmup_steps=0, quantize_coefficients=True)
    codec = CheckpointBoundaryCodec(spec).cuda()
    base = torch.randn(4 * 128, rank, device="cuda", generator=g) @ torch.randn(rank, hidden, device="cuda", generator=g)
    x = (base + 0.01 * torch.randn(4 * 128, hidden, device="cuda", generator=g)).bfloat16().reshape(4, 128, hidden)
    rec = codec.pack_tensor(x, training=True)
    assert not rec.is_dense_fallback and rec.coeff.dtype == torch.int8
    back = codec.unpack_record(rec)
    assert back.shape == x.shape and back.dtype == torch.bfloat16
    rel = float((back.float() - x.float()).norm() / x.float().norm())
    assert rel < 0.05, rel
