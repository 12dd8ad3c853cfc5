"""Fused forward primitives: framework route on CPU, kernel route on a B200."""

import pytest
import torch

from stacr_b200 import fused_kernels as FK


@pytest.mark.parametrize("mode", ["row", "global"])
def test_chunked_route_matches_the_unchunked_reference(mode):
    torch.manual_seed(0)
    x = torch.randn(50, 64)
    q = torch.linalg.qr(torch.randn(64, 8)).Q
    c, v, i, meta = FK.stacr_forward_fused(x, q, 0.1, mode, chunk_size=16, return_metadata=True)
    c0, v0, i0 = FK.stacr_forward_pytorch(x, q.t(), 0.1, mode)           # the basis may come as [R, N] too
    torch.testing.assert_close(c, c0, rtol=1e-5, atol=1e-6)
    assert meta["route"] == "pytorch_chunked" and meta["route_counts"]["pytorch_chunked"] == 4
    if mode == "row":
        assert v.shape == (50, 6) and torch.equal(i.sort(dim=1).values, i0.sort(dim=1).values)
    else:
        assert v.shape == (320,) and set(i.tolist()) == set(i0.tolist())
        dense = x - (x @ q) @ q.t()
        torch.testing.assert_close(v, dense.reshape(-1)[i], rtol=1e-5, atol=1e-6)    # values keep their sign


def test_argument_checks_and_aliases():
    x, q = torch.randn(4, 16), torch.randn(16, 2)
    with pytest.raises(ValueError):
        FK.stacr_forward_fused(x, torch.randn(5, 3))
    with pytest.raises(ValueError):
        FK.stacr_forward_fused(x, q, topk_mode="column")
    with pytest.raises(ValueError):
        FK.triton_matmul(x, torch.randn(3, 3))
    torch.testing.assert_close(FK.triton_matmul(x, q), x @ q)
    import stacr.triton_kernels as alias
    from stacr_b200 import triton_kernels

    assert alias.stacr_forward_fused is FK.stacr_forward_fused and triton_kernels.triton_matmul is FK.triton_matmul
    assert FK.verify_fused_kernel(B=16, N=64, R=4, budget=0.2, topk_mode="global")


@pytest.mark.gpu
def test_kernel_route_selects_the_same_entries_as_the_reference():
    torch.manual_seed(1)
    x = (torch.randn(512, 8, device="cuda") @ torch.randn(8, 1024, device="cuda") + 0.5 * torch.randn(512, 1024, device="cuda")).bfloat16()
    q = torch.linalg.qr(torch.randn(1024, 8, device="cuda")).Q.bfloat16()
    c, v, i, meta = FK.stacr_forward_fused(x, q, 0.01, "global", return_metadata=True)
    assert meta["route"] == "sm100_kernels" and i.dtype == torch.int64 and v.numel() == int(512 * 1024 * 0.01)
    coeff = (x.float() @ q.float())
    torch.testing.assert_close(c.float(), coeff, rtol=2e-2, atol=2e-2)
    res = (x.float() - c.float() @ q.float().t()).bfloat16().float().reshape(-1)    # the residual the kernels see
    kth = res.abs().topk(v.numel()).values[-1]
    assert float(res[i].abs().min()) >= float(kth) * 0.99                            # only entries at or above the k-th magnitude
    torch.testing.assert_close(v.float(), res[i], rtol=2e-2, atol=2e-2)
    y = FK.triton_matmul(x, q)
    torch.testing.assert_close(y.float(), coeff, rtol=2e-2, atol=5e-2)
