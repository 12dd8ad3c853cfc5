"""Index arithmetic of device kernels restated on the host and checked exhaustively (no GPU needed).

Each emulation follows its kernel statement by statement; what is asserted is the property the kernel relies on, so a change to
one of the constants in the kernel has to be mirrored here and re-proved.
"""

import itertools

import torch


# ---- basis.cu: cluster_gram8 -- a warp reduce-scatter of 36 per-lane partial sums in 18 + 9 + 5 + 3 + 2 = 37 shuffles
def _scatter_round(values, n_out, off):
    """``values[lane]`` is that lane's list; lanes with bit ``off`` clear keep the first ``n_out`` entries, the others the rest,
    each adding what its partner ``lane ^ off`` held of the kept half (missing entries count as zero)."""
    n_in = len(values[0])
    out = []
    for lane in range(32):
        hi = bool(lane & off)
        mine, partner = values[lane], values[lane ^ off]
        row = []
        for i in range(n_out):
            pick = (lambda v: (v[i + n_out] if i + n_out < n_in else 0.0)) if hi else (lambda v: v[i])
            row.append(pick(mine) + pick(partner))
        out.append(row)
    return out


def test_gram_butterfly_delivers_every_sum_exactly_once():
    torch.manual_seed(0)
    acc = torch.randn(32, 36, dtype=torch.float64)
    v = [list(map(float, acc[lane])) for lane in range(32)]
    for n_out, off in ((18, 16), (9, 8), (5, 4), (3, 2), (2, 1)):
        v = _scatter_round(v, n_out, off)
    landed = [0.0] * 36
    hits = [0] * 36
    for lane in range(32):
        b4, b3, b2, b1, b0 = (lane >> 4) & 1, (lane >> 3) & 1, (lane >> 2) & 1, (lane >> 1) & 1, lane & 1
        l3 = 4 if b2 else 5
        l4 = l3 - 3 if b1 else 3
        l5 = l4 - 2 if b0 else min(l4, 2)
        base = 18 * b4 + 9 * b3 + 5 * b2 + 3 * b1 + 2 * b0
        for slot in range(2):
            if slot < l5:
                landed[base + slot] += v[lane][slot]
                hits[base + slot] += 1
    assert hits == [1] * 36                                    # no sum is dropped, none is counted twice
    torch.testing.assert_close(torch.tensor(landed, dtype=torch.float64), acc.sum(0))


def test_gram_triangle_index_decoding():
    """The 36 sums are the lower triangle of an 8 x 8 Gram matrix, row by row; thread t decodes (i, j) with a running base."""
    seen = {}
    for t in range(36):
        i, base = 0, 0
        while base + i + 1 <= t:
            base += i + 1
            i += 1
        seen[t] = (i, t - base)
    assert list(seen.values()) == [(i, j) for i in range(8) for j in range(i + 1)]


# ---- attention.cu / ops/attention.py: addressing of q, k, v inside a fused projection output
def test_fused_qkv_views_address_the_projection_output_in_place():
    from stacr_b200.ops import attention

    b, s, h, d = 2, 5, 3, 8
    qkv = torch.arange(b * s * 3 * h * d, dtype=torch.float32).view(b * s, 3 * h * d)
    for layout in ("interleaved", "blocked"):
        views = attention.qkv_views(qkv, b, s, h, d, layout)
        for which, t in enumerate(views):
            assert t.shape == (b, h, s, d)
            ld, head_stride = t.stride(2), t.stride(1)
            col0 = (t.data_ptr() - qkv.data_ptr()) // qkv.element_size()
            for bi, hi, si in itertools.product(range(b), range(h), range(s)):
                # the kernels' address: base + (b * S + s) * ld + col0 + h * head_stride
                flat = (bi * s + si) * ld + col0 + hi * head_stride
                assert torch.equal(qkv.flatten()[flat:flat + d], t[bi, hi, si])
            expected_col0 = which * d if layout == "interleaved" else which * h * d
            assert col0 == expected_col0 and head_stride == (3 * d if layout == "interleaved" else d)


# ---- stacr_select.cu: per-chunk quota of the allocation-free entry point (rounded share of the last, shorter chunk)
def test_noalloc_chunk_quota_formula_matches_its_host_twin():
    from stacr_b200.ops import _lib

    if not _lib.available():
        return
    lib = _lib.load()
    import ctypes

    lib.sb_residual_topk_noalloc_count.restype = ctypes.c_longlong
    for rows, chunk, quota in itertools.product((1, 7, 512, 1000, 4096), (1, 64, 512), (0, 1, 13, 700)):
        total = 0
        for c in range((rows + chunk - 1) // chunk):
            length = min(chunk, rows - c * chunk)
            total += quota if length == chunk else max(1, (quota * length + chunk // 2) // chunk)   # a partial chunk keeps >= 1
        assert lib.sb_residual_topk_noalloc_count(ctypes.c_int(rows), ctypes.c_int(chunk), ctypes.c_int(quota)) == total
