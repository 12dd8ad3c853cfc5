"""The allocation-free residual selection entry point against the regular one.

Some users of the kernel library may not allocate device memory at the point where they call it:
a step that is being recorded into a CUDA graph, a training loop whose memory peak was planned in
advance and must not grow the allocator's pool, or a host application that lends the library a
fixed arena and bans cudaMalloc/cudaFree because they stall the whole device.  For them the
library exports ``sb_residual_topk_noalloc``, whose histogram and counters live in a device array
built into the library instead of in buffers the caller allocates.  This test drives that symbol
through ctypes, exactly as such a caller would, and requires the same selection as the regular
entry point on two consecutive calls (the second one with a different shape and chunking, so that
anything the first call left in the shared scratch would show).
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(rows, n, r, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    low = torch.randn(rows, r, device="cuda", generator=g) @ torch.randn(r, n, device="cuda", generator=g)
    x = (low + 0.3 * torch.randn(rows, n, device="cuda", generator=g)).bfloat16()
    qb = torch.linalg.qr(torch.randn(n, r, device="cuda", generator=g)).Q.bfloat16().contiguous()
    c = (x.float() @ qb.float()).bfloat16().contiguous()
    e = (x.float() - c.float() @ qb.float().t()).bfloat16().reshape(-1)
    return x, qb, c, e


def _call_noalloc(lib, x, c, qb, chunk_rows, quota, bits):
    from stacr_b200.ops import _lib

    rows, n = x.shape
    lib.sb_residual_topk_noalloc_count.restype = ctypes.c_longlong
    total = lib.sb_residual_topk_noalloc_count(ctypes.c_int(rows), ctypes.c_int(chunk_rows), ctypes.c_int(quota))
    assert total > 0
    # outputs are the caller's; everything else the call needs is inside the library
    idx = torch.empty(total, dtype=torch.int32, device="cuda")
    val = torch.empty(total, dtype=torch.bfloat16 if bits == 0 else torch.int8, device="cuda")
    scale = torch.empty((), dtype=torch.float32, device="cuda")
    status = _lib.status_word()  # created once per device by the binding; not part of the call under test
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = lib.sb_residual_topk_noalloc(
        _lib.ptr(x), _lib.ptr(c), _lib.ptr(qb), ctypes.c_int(rows), ctypes.c_int(n), ctypes.c_int(c.shape[1]), ctypes.c_int(x.stride(0)),
        ctypes.c_int(chunk_rows), ctypes.c_int(quota), ctypes.c_int(bits), _lib.ptr(idx), ctypes.c_void_p(0), _lib.ptr(val),
        _lib.ptr(scale), _lib.ptr(status), _lib.stream_ptr(),
    )
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    _lib.check_status()
    return idx, val, scale


def _same_selection(e, n, chunk_rows, idx_a, val_a, scale_a, idx_b, val_b, scale_b, bits):
    assert idx_a.numel() == idx_b.numel()
    assert idx_a.unique().numel() == idx_a.numel()
    torch.testing.assert_close(scale_a, scale_b, rtol=0, atol=0)
    mag_a = e[idx_a.long()].float().abs()
    mag_b = e[idx_b.long()].float().abs()
    chunk_a = (idx_a.long() // n) // chunk_rows
    chunk_b = (idx_b.long() // n) // chunk_rows
    for ch in chunk_b.unique().tolist():
        sa, sb = mag_a[chunk_a == ch].sort().values, mag_b[chunk_b == ch].sort().values
        # same tolerance as the selection tests of the regular entry point: one bf16 ulp at the threshold
        torch.testing.assert_close(sa, sb, rtol=2e-2, atol=1e-3)
    # values travel with their indices in both outputs
    order_a, order_b = idx_a.long().argsort(), idx_b.long().argsort()
    common = idx_a.long()[order_a] == idx_b.long()[order_b]
    va = val_a.float()[order_a][common] * (scale_a if bits else 1.0)
    vb = val_b.float()[order_b][common] * (scale_b if bits else 1.0)
    torch.testing.assert_close(va, vb, rtol=2e-2, atol=1e-3)


def test_noalloc_entry_matches_regular_entry_on_two_consecutive_calls():
    from stacr_b200.ops import _lib, stacr_ops

    lib = _lib.load()
    assert hasattr(lib, "sb_residual_topk_noalloc")
    # call 1: four chunks of 256 rows, int8 codes
    x, qb, c, e = _case(1024, 1024, 8, seed=1)
    quota = int(round(0.01 * 256 * 1024))
    got = _call_noalloc(lib, x, c, qb, 256, quota, 8)
    ref = stacr_ops.residual_topk(x, c, qb, [quota] * 4, 256, 8, torch.int32)
    torch.cuda.synchronize()
    _same_selection(e, 1024, 256, *got, *ref, bits=8)
    # call 2 straight after: one global chunk, other shape, raw bf16 values
    x, qb, c, e = _case(768, 2048, 8, seed=2)
    quota = int(round(0.004 * 768 * 2048))
    got = _call_noalloc(lib, x, c, qb, 768, quota, 0)
    ref = stacr_ops.residual_topk(x, c, qb, [quota], 768, 0, torch.int32)
    torch.cuda.synchronize()
    _same_selection(e, 2048, 768, *got, *ref, bits=0)


def test_noalloc_entry_rejects_requests_beyond_its_scratch():
    from stacr_b200.ops import _lib

    lib = _lib.load()
    x, qb, c, _ = _case(1024, 256, 8, seed=3)
    idx = torch.empty(64, dtype=torch.int32, device="cuda")
    val = torch.empty(64, dtype=torch.int8, device="cuda")
    scale = torch.empty((), dtype=torch.float32, device="cuda")
    rc = lib.sb_residual_topk_noalloc(  # 1024 rows in chunks of 32 rows = 32 chunks > 16
        _lib.ptr(x), _lib.ptr(c), _lib.ptr(qb), ctypes.c_int(1024), ctypes.c_int(256), ctypes.c_int(8), ctypes.c_int(256),
        ctypes.c_int(32), ctypes.c_int(2), ctypes.c_int(8), _lib.ptr(idx), ctypes.c_void_p(0), _lib.ptr(val), _lib.ptr(scale),
        _lib.ptr(_lib.status_word()), _lib.stream_ptr(),
    )
    assert rc == -7


def test_noalloc_entry_rejects_a_quota_larger_than_a_chunk():
    from stacr_b200.ops import _lib

    lib = _lib.load()
    x, qb, c, _ = _case(64, 64, 8, seed=4)
    idx = torch.empty(8192, dtype=torch.int32, device="cuda")
    val = torch.empty(8192, dtype=torch.int8, device="cuda")
    scale = torch.empty((), dtype=torch.float32, device="cuda")
    rc = lib.sb_residual_topk_noalloc(  # a chunk of 32 rows x 64 columns has 2048 entries; 4096 are asked for
        _lib.ptr(x), _lib.ptr(c), _lib.ptr(qb), ctypes.c_int(64), ctypes.c_int(64), ctypes.c_int(8), ctypes.c_int(64),
        ctypes.c_int(32), ctypes.c_int(4096), ctypes.c_int(8), _lib.ptr(idx), ctypes.c_void_p(0), _lib.ptr(val), _lib.ptr(scale),
        _lib.ptr(_lib.status_word()), _lib.stream_ptr(),
    )
    assert rc == -2
