"""Python entry points for the compressed-linear kernels (projection, selection, basis, dW)."""

from __future__ import annotations

import os

import ctypes
import math

import torch

from . import _lib
from .gemm import gemm

c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


def rank_pad(rank: int) -> int:
    """Width of the padded rank panel the tensor-core kernels use (UMMA N is a multiple of 16)."""
    return 16 if rank <= 16 else 32


def pad_basis_transpose(basis_bf16: torch.Tensor) -> torch.Tensor:
    """``[N, r]`` bf16 basis -> zero-padded ``[rpad, N]`` K-major panel."""
    n, r = basis_bf16.shape
    out = torch.zeros(rank_pad(r), n, dtype=torch.bfloat16, device=basis_bf16.device)
    out[:r] = basis_bf16.t()
    return out


def _splits_for(m_rows: int, k: int, device) -> int:
    tiles = (m_rows + 127) // 128
    kb = (k + 63) // 64
    return max(1, min(kb, _lib.sm_count(device) // max(1, tiles)))


def project(x: torch.Tensor, qt_pad: torch.Tensor) -> torch.Tensor:
    """``X[rows, N] @ Q`` with the padded transposed basis ``[rpad, N]``; fp32 ``[rows, rpad]``."""
    rows, n = x.shape
    return gemm(x, qt_pad, splits=max(2, _splits_for(rows, n, x.device)), bn=qt_pad.shape[0])


def at_b(a: torch.Tensor, bt_pad: torch.Tensor) -> torch.Tensor:
    """``A[rows, M]^T @ B`` where ``bt_pad`` is the padded transpose ``[rpad, rows]``; fp32 ``[M, rpad]``."""
    rows, m = a.shape
    return gemm(a, bt_pad, a_mn=True, splits=max(2, _splits_for(m, rows, a.device)), bn=bt_pad.shape[0])


def transpose_pad(c: torch.Tensor) -> torch.Tensor:
    """``[rows, r]`` (bf16 or fp32) -> zero-padded bf16 ``[rpad, rows]``."""
    rows, r = c.shape
    out = torch.zeros(rank_pad(r), rows, dtype=torch.bfloat16, device=c.device)
    out[:r] = c.t()
    return out


_META: dict = {}
_NBINS = 32768
_SAMPLE_STRIDE = 16


def _sampled_ok(quotas: list[int], rows: int, n: int, chunk_rows: int) -> bool:
    """Whether every chunk is large and sparse enough for the sampled-threshold selection to pay off."""
    if os.environ.get("STACR_SELECT_SAMPLED", "1") != "1" or n < 64 or n % 8:
        return False
    for i, k in enumerate(quotas):
        elems = (min(rows, (i + 1) * chunk_rows) - i * chunk_rows) * n
        if elems < (1 << 19) or k < 1024 or k * 8 > elems:
            return False
    return True


def _select_meta(dev, quotas: list[int], sampled: bool):
    """Per-chunk quotas, output offsets and (sampled form) candidate-list layout, uploaded once per distinct schedule."""
    key = (dev.index, tuple(quotas), sampled)
    meta = _META.get(key)
    if meta is None:
        offsets = [0]
        for k in quotas[:-1]:
            offsets.append(offsets[-1] + k)
        rows_i = [quotas, offsets]
        margins, total_cap = [], 0
        if sampled:
            caps, coffs = [], []
            for k in quotas:
                margin = min(3.0, max(1.25, 1.0 + 8.0 / math.sqrt(max(1.0, k / _SAMPLE_STRIDE))))
                cap = int(1.5 * margin * k) + 8192
                margins.append(margin)
                coffs.append(total_cap)
                caps.append(cap)
                total_cap += cap
            rows_i += [coffs, caps]
        meta = {"ints": torch.tensor(rows_i, dtype=torch.int32).to(dev), "cap": total_cap, "max_cap": max(caps) if sampled else 0,
                "margin": torch.tensor(margins, dtype=torch.float32).to(dev) if sampled else None}
        if len(_META) > 256:
            _META.clear()
        _META[key] = meta
    return meta


def residual_topk(
    x: torch.Tensor,
    coeff: torch.Tensor,
    basis_bf16: torch.Tensor,
    quotas: list[int],
    chunk_rows: int,
    bits: int,
    index_dtype: torch.dtype,
    sampled: bool | None = None,
):
    """Exact per-chunk top-k of ``|X - C Q^T|``; returns ``(idx, values, scale)``.

    ``values`` are bf16 (``bits == 0``) or int8 holding the 8- or 4-bit codes; ``scale`` is an
    fp32 scalar tensor.  Entry order is unspecified.  ``sampled`` picks the one-pass form (threshold
    estimated from a 1/16 sample, exact selection among the candidates above it, exact two-pass redo of
    any chunk the sample misjudged); ``None`` uses it when every chunk is large and sparse enough.
    """
    rows, n = x.shape
    r = coeff.shape[1]
    nchunks = len(quotas)
    dev = x.device
    total = sum(quotas)
    sms = _lib.sm_count(dev)
    parts = max(1, sms // nchunks)
    if sampled is None:
        sampled = _sampled_ok(quotas, rows, n, chunk_rows)
    meta = _select_meta(dev, quotas, sampled)
    ints = meta["ints"]
    idx = torch.empty(total, dtype=index_dtype, device=dev)
    val = torch.empty(total, dtype=torch.bfloat16 if bits == 0 else torch.int8, device=dev)
    scale = torch.empty((), dtype=torch.float32, device=dev)
    is32 = index_dtype == torch.int32
    lib = _lib.load()
    if sampled:
        # two histograms, the per-chunk counters and two global words: one fill
        scratch = torch.zeros(nchunks * (2 * _NBINS + 12) + 2, dtype=torch.int32, device=dev)
        hist, hist2, work = scratch[: nchunks * _NBINS], scratch[nchunks * _NBINS: 2 * nchunks * _NBINS], scratch[2 * nchunks * _NBINS:]
        cand_idx = torch.empty(meta["cap"], dtype=torch.int64, device=dev)
        cand_val = torch.empty(meta["cap"], dtype=torch.int16, device=dev)
        rc = lib.sb_residual_topk_sampled(
            _lib.ptr(x), _lib.ptr(coeff), _lib.ptr(basis_bf16), c_int(rows), c_int(n), c_int(r), c_int(x.stride(0)), c_int(chunk_rows),
            c_int(nchunks), c_int(parts), _lib.ptr(hist), _lib.ptr(hist2), _lib.ptr(work), _lib.ptr(ints[0]), _lib.ptr(ints[1]),
            _lib.ptr(ints[2]), _lib.ptr(ints[3]), _lib.ptr(meta["margin"]), _lib.ptr(cand_idx), _lib.ptr(cand_val), c_int(meta["max_cap"]), c_int(bits),
            _lib.ptr(idx if is32 else None), _lib.ptr(None if is32 else idx), _lib.ptr(val), _lib.ptr(scale),
            _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_residual_topk_sampled")
        _lib.count(6)
        global _LAST_SAMPLED_WORK
        _LAST_SAMPLED_WORK = (work, nchunks)
        return idx, val, scale
    scratch = torch.zeros(nchunks * (_NBINS + 6), dtype=torch.int32, device=dev)   # histogram and counters: one fill
    hist, work = scratch[: nchunks * _NBINS], scratch[nchunks * _NBINS:]
    rc = lib.sb_residual_topk(
        _lib.ptr(x), _lib.ptr(coeff), _lib.ptr(basis_bf16), c_int(rows), c_int(n), c_int(r), c_int(x.stride(0)),
        c_int(chunk_rows), c_int(nchunks), c_int(parts), _lib.ptr(hist), _lib.ptr(work), _lib.ptr(ints[0]), _lib.ptr(ints[1]),
        c_int(bits), _lib.ptr(idx if is32 else None), _lib.ptr(None if is32 else idx), _lib.ptr(val), _lib.ptr(scale),
        _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "sb_residual_topk")
    _lib.count(4)
    return idx, val, scale


_ABOVE_CAP: dict = {}


def residual_above(x: torch.Tensor, coeff: torch.Tensor, basis_bf16: torch.Tensor, threshold: float):
    """Flat indices (int64) and bf16 values of the residual entries with ``|e| > threshold``: one pass over ``X``.

    The number of hits is data dependent, so the call ends with a host read of one counter (as ``nonzero`` would); the list
    capacity is remembered per shape from call to call and the pass is repeated once when it proves too small.
    """
    rows, n = x.shape
    dev = x.device
    if n % 8:
        e = (x.float() - coeff.float() @ basis_bf16.float().t()).to(torch.bfloat16).reshape(-1)
        idx = (e.float().abs() > threshold).nonzero(as_tuple=True)[0]
        return idx, e[idx]
    key = (dev.index, rows, n)
    cap = _ABOVE_CAP.get(key, max(4096, rows * n // 64))
    cut = max(0.0, float(threshold) * (1.0 - 2.0 ** -7))      # every value whose bf16 rounding can exceed the threshold
    lib = _lib.load()
    parts = _lib.sm_count(dev)
    while True:
        scratch = torch.zeros(2 * _NBINS + 14, dtype=torch.int32, device=dev)
        hist, hist2, work = scratch[:_NBINS], scratch[_NBINS: 2 * _NBINS], scratch[2 * _NBINS:]
        meta = torch.tensor([0, 0, 0, cap], dtype=torch.int32).to(dev)
        cand_idx = torch.empty(cap, dtype=torch.int64, device=dev)
        cand_val = torch.empty(cap, dtype=torch.bfloat16, device=dev)
        scale = torch.empty((), dtype=torch.float32, device=dev)
        rc = lib.sb_residual_above(
            _lib.ptr(x), _lib.ptr(coeff), _lib.ptr(basis_bf16), c_int(rows), c_int(n), c_int(coeff.shape[1]), c_int(x.stride(0)), c_float(cut),
            c_int(parts), _lib.ptr(hist), _lib.ptr(hist2), _lib.ptr(work), _lib.ptr(meta), _lib.ptr(cand_idx), _lib.ptr(cand_val), _lib.ptr(scale),
            _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_residual_above")
        _lib.count(1)
        found = int(work[6].item())
        if found <= cap:
            break
        cap = int(found * 1.25) + 1024
    _ABOVE_CAP[key] = max(4096, int(found * 1.5))
    idx, val = cand_idx[:found], cand_val[:found]
    keep = val.float().abs() > threshold
    return idx[keep], val[keep]


_LAST_SAMPLED_WORK = None


def last_sampled_selection_stats() -> dict | None:
    """Counters of the most recent sampled selection (a synchronising read, for tests and diagnostics): per chunk the
    candidate bin, the number of candidates the full pass appended and whether the chunk was redone by the exact passes."""
    if _LAST_SAMPLED_WORK is None:
        return None
    work, n = _LAST_SAMPLED_WORK
    host = work.cpu()
    return {"candidate_bin": host[5 * n: 6 * n].tolist(), "candidates": host[6 * n: 7 * n].tolist(), "fell_back": host[7 * n: 8 * n].tolist()}


def residual_gather(x, coeff, basis_bf16, idx: torch.Tensor) -> torch.Tensor:
    """bf16 residual values at explicit flat indices."""
    n, r = basis_bf16.shape
    out = torch.empty(idx.numel(), dtype=torch.bfloat16, device=x.device)
    is32 = idx.dtype == torch.int32
    rc = _lib.load().sb_residual_gather(
        _lib.ptr(x), _lib.ptr(coeff), _lib.ptr(basis_bf16), c_int(n), c_int(r), c_int(x.stride(0)),
        _lib.ptr(None if is32 else idx), _lib.ptr(idx if is32 else None), c_ll(idx.numel()), _lib.ptr(out), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "sb_residual_gather")
    _lib.count(1)
    return out


def residual_block_energy(x, coeff, basis_bf16, block: int) -> torch.Tensor:
    rows, n = x.shape
    out = torch.empty(rows, n // block, dtype=torch.float32, device=x.device)
    rc = _lib.load().sb_residual_block_energy(
        _lib.ptr(x), _lib.ptr(coeff), _lib.ptr(basis_bf16), c_int(rows), c_int(n), c_int(coeff.shape[1]), c_int(x.stride(0)),
        c_int(block), _lib.ptr(out), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "sb_residual_block_energy")
    _lib.count(1)
    return out


def oja_update(basis_fp32, g, y, rows: int, lr: float):
    """One fused Oja + CholeskyQR2 step; returns ``(basis_fp32, basis_bf16, basis_t_pad_bf16)``.

    ``g`` is ``X^T Y`` ``[N, >=r]`` fp32 and ``y`` is ``[rows, >=r]`` fp32; pass ``None`` for both
    (and ``lr=0``) to only re-orthonormalise.
    """
    n, r = basis_fp32.shape
    dev = basis_fp32.device
    q_in = basis_fp32.contiguous()
    q_out = torch.empty_like(q_in)
    qb = torch.empty(n, r, dtype=torch.bfloat16, device=dev)
    rp = rank_pad(r)
    qt = torch.empty(rp, n, dtype=torch.bfloat16, device=dev)
    rc = _lib.load().sb_oja_update(
        _lib.ptr(q_in), _lib.ptr(g), c_int(0 if g is None else g.stride(0)), _lib.ptr(y), c_int(0 if y is None else y.stride(0)),
        c_int(rows), c_int(n), c_int(r), c_float(lr if g is not None else 0.0), _lib.ptr(q_out), _lib.ptr(qb), _lib.ptr(qt),
        c_int(rp), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "sb_oja_update")
    _lib.count(1)
    return q_out, qb, qt


def orthonormalize_columns_(a: torch.Tensor) -> torch.Tensor:
    """In-place orthonormalisation of the columns of a contiguous fp32 ``[n, w]`` matrix, ``w <= 32`` (Gram-Schmidt with
    re-orthogonalisation in one kernel: robust for the nearly collinear iterates of a subspace iteration)."""
    assert a.dtype == torch.float32 and a.dim() == 2 and a.is_contiguous() and a.shape[1] <= 32
    rc = _lib.load().sb_mgs_qr(_lib.ptr(a), c_int(a.shape[0]), c_int(a.shape[1]), c_int(a.stride(0)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_mgs_qr")
    _lib.count(1)
    return a


def small_gram(a: torch.Tensor) -> torch.Tensor:
    """fp64 ``a^T a`` of a contiguous fp32 ``[rows, w]`` matrix, ``w <= 32``."""
    assert a.dtype == torch.float32 and a.dim() == 2 and a.stride(1) == 1 and a.shape[1] <= 32
    w = a.shape[1]
    out = torch.zeros(w, w, dtype=torch.float64, device=a.device)
    rc = _lib.load().sb_gram_small(_lib.ptr(a), c_int(a.shape[0]), c_int(w), c_int(a.stride(0)), _lib.ptr(out), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_gram_small")
    _lib.count(1)
    return out


def small_eigh(m: torch.Tensor):
    """``(eigenvalues descending, eigenvectors in columns)`` of a symmetric fp64 matrix of order ``<= 32`` (cyclic Jacobi)."""
    assert m.dtype == torch.float64 and m.dim() == 2 and m.shape[0] == m.shape[1] <= 32
    m = m.contiguous()
    w = m.shape[0]
    evals = torch.empty(w, dtype=torch.float64, device=m.device)
    evecs = torch.empty(w, w, dtype=torch.float64, device=m.device)
    rc = _lib.load().sb_jacobi_eig(_lib.ptr(m), c_int(w), _lib.ptr(evals), _lib.ptr(evecs), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_jacobi_eig")
    _lib.count(1)
    return evals, evecs


_PLAN_TARGET = None


def _plan_target() -> int:
    global _PLAN_TARGET
    if _PLAN_TARGET is None:
        _PLAN_TARGET = int(_lib.load().sb_dw_plan_target())
    return _PLAN_TARGET


_REBUILD: dict = {}


def _dense_threshold() -> int:
    """Smallest ``rows * in_features * out_features`` for which the weight gradient is formed as a dense tensor-core product
    of ``dY`` with the transiently rebuilt input (``STACR_DW_DENSE_MIN``, default 2**33; 0 = always, -1 = never)."""
    return int(os.environ.get("STACR_DW_DENSE_MIN", str(1 << 33)))


def rebuild_input(coeff: torch.Tensor, basis_fp32: torch.Tensor, residual, rows: int, in_features: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """``bf16(C Q^T + S)``, written into ``out`` (contiguous bf16 ``[rows, in_features]``) or, without one, into a per-shape
    scratch buffer that later calls overwrite (valid until the next call of this shape)."""
    dev = coeff.device
    key = (dev.index, rows, in_features)
    buf = out if out is not None else _REBUILD.get(key)
    if out is not None:
        assert out.dtype == torch.bfloat16 and out.is_contiguous() and tuple(out.shape) == (rows, in_features)
    if buf is None:
        if len(_REBUILD) > 8:
            _REBUILD.clear()
        buf = torch.empty(rows, in_features, dtype=torch.bfloat16, device=dev)
        _REBUILD[key] = buf
    idx = values = scale = None
    bits, length = 0, 0
    if residual is not None and residual[4] > 0:
        idx, values, scale, bits, length = residual
    is32 = idx is not None and idx.dtype == torch.int32
    rc = _lib.load().sb_rebuild_input(
        _lib.ptr(coeff), _lib.ptr(basis_fp32), c_int(coeff.shape[1]), c_int(rows), c_int(in_features), _lib.ptr(idx if is32 else None),
        _lib.ptr(None if (is32 or idx is None) else idx), c_ll(length), _lib.ptr(values), c_int(int(bits)), _lib.ptr(scale), _lib.ptr(buf),
        c_int(in_features), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "sb_rebuild_input")
    _lib.count(2 if length else 1)
    return buf


def weight_grad(
    dy: torch.Tensor,
    coeff: torch.Tensor,
    basis_fp32: torch.Tensor,
    residual,
    out_features: int,
    in_features: int,
    transposed: bool,
    out_dtype: torch.dtype,
    sink=None,
    out: torch.Tensor | None = None,
    dense: bool | None = None,
):
    """``dW = (dY^T C) Q^T + dY^T S`` from the saved factors.

    Two forms.  The gather form never rebuilds the input: a skinny GEMM gives ``dY^T C``, the residual is bucketed by feature
    and one kernel expands the rank-r term and gathers ``dY`` rows.  The dense form (``dense=True``; chosen automatically for
    large layers that carry a residual, see ``_dense_threshold``) rebuilds ``bf16(C Q^T + S)`` in a scratch buffer for the
    duration of the call and runs one tensor-core GEMM with ``dY``; what is saved between forward and backward is the same.

    ``residual`` is ``None`` or ``(idx, values, scale, bits, length)``.  With ``sink`` (see
    ``parallel.ddp.GradSink``) the gradient is not returned: the kernel adds it straight into the flat gradient
    buffer, or, across data-parallel ranks, into the copy of the rank that owns each slice (reduce-scatter in the
    epilogue over NVLink peer memory); the function then returns ``None``.
    """
    dev = dy.device
    rows = dy.shape[0]
    r = coeff.shape[1]
    has_residual = residual is not None and residual[4] > 0
    if dense is None:
        floor = _dense_threshold()
        dense = has_residual and sink is None and floor >= 0 and rows * in_features * out_features >= floor
    if dense and sink is None and dy.stride(1) == 1 and dy.stride(0) % 8 == 0 and in_features % 8 == 0 and out_features % 8 == 0 \
            and basis_fp32.dtype == torch.float32 and basis_fp32.is_contiguous() and coeff.is_contiguous():
        # large layer with a residual: one dense product on the tensor cores with the input rebuilt for this call only
        xhat = rebuild_input(coeff, basis_fp32, residual, rows, in_features)
        shape = (in_features, out_features) if transposed else (out_features, in_features)
        if out is None:
            out = torch.empty(shape, dtype=out_dtype, device=dev)
        else:
            assert out.shape == shape and out.dtype == out_dtype and out.is_contiguous()
        if transposed:
            return gemm(xhat, dy, a_mn=True, b_mn=True, out=out, out_dtype=out_dtype)
        return gemm(dy, xhat, a_mn=True, b_mn=True, out=out, out_dtype=out_dtype)
    t = at_b(dy, transpose_pad(coeff))  # [O, rpad] fp32
    colptr = rows_s = vals_s = plan = None
    nnz = 0
    if residual is not None and residual[4] > 0:
        idx, values, scale, bits, length = residual
        counts = torch.zeros(in_features, dtype=torch.int32, device=dev)
        cursor = torch.empty(in_features, dtype=torch.int32, device=dev)
        colptr = torch.empty(in_features + 1, dtype=torch.int32, device=dev)
        rows_s = torch.empty(length, dtype=torch.int32, device=dev)
        vals_s = torch.empty(length, dtype=torch.float32, device=dev)
        groups = (in_features + 7) // 8
        # work plan of the gradient kernel: pieces per strip of 8 features, item count, (strip, piece) items
        plan = torch.empty(groups + 2 + 2 * (length // _plan_target()), dtype=torch.int32, device=dev)
        nnz = length
        is32 = idx.dtype == torch.int32
        rc = _lib.load().sb_residual_bucket(
            _lib.ptr(idx if is32 else None), _lib.ptr(None if is32 else idx), c_ll(length), c_int(in_features), _lib.ptr(values),
            c_int(bits), _lib.ptr(scale), _lib.ptr(counts), _lib.ptr(cursor), _lib.ptr(colptr), _lib.ptr(rows_s), _lib.ptr(vals_s),
            _lib.ptr(plan), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_residual_bucket")
        _lib.count(3)
    if sink is not None:
        rc = _lib.load().sb_dw_fused_sink(
            _lib.ptr(t), c_int(t.stride(0)), _lib.ptr(basis_fp32), c_int(r), _lib.ptr(dy), c_int(dy.stride(0)), _lib.ptr(colptr),
            _lib.ptr(rows_s), _lib.ptr(vals_s), c_int(out_features), c_int(in_features), c_int(int(transposed)), _lib.ptr(sink.flat),
            c_int(sink.mode), ctypes.c_float(sink.scale), c_ll(sink.param_off), c_ll(sink.region_lo), c_ll(sink.per_vecs), c_int(sink.world),
            _lib.ptr(sink.peer_ptrs), _lib.ptr(plan), c_ll(nnz), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_dw_fused_sink")
        _lib.count(2 if nnz >= _plan_target() else 1)
        return None
    shape = (in_features, out_features) if transposed else (out_features, in_features)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=dev)
    else:  # the caller's buffer (for example the parameter's slot of a flat gradient buffer) is written directly
        assert out.shape == shape and out.dtype == out_dtype and out.is_contiguous()
    rc = _lib.load().sb_dw_fused(
        _lib.ptr(t), c_int(t.stride(0)), _lib.ptr(basis_fp32), c_int(r), _lib.ptr(dy), c_int(dy.stride(0)), _lib.ptr(colptr),
        _lib.ptr(rows_s), _lib.ptr(vals_s), c_int(out_features), c_int(in_features), c_int(int(transposed)),
        c_int(int(out_dtype == torch.bfloat16)), _lib.ptr(out), _lib.ptr(plan), c_ll(nnz), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "sb_dw_fused")
    _lib.count(2 if (nnz >= _plan_target() and out_dtype != torch.bfloat16) else 1)
    return out


def colsum(dy: torch.Tensor) -> torch.Tensor:
    rows, o = dy.shape
    out = torch.zeros(o, dtype=torch.float32, device=dy.device)
    rc = _lib.load().sb_colsum_bf16(_lib.ptr(dy), c_int(rows), c_int(o), c_int(dy.stride(0)), _lib.ptr(out), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_colsum_bf16")
    _lib.count(1)
    return out
