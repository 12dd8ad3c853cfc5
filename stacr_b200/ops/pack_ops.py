"""Python entry points for ``csrc/index_pack.cu``: index-stream encodings, per-tensor codecs, row moves."""

from __future__ import annotations

import ctypes

import torch

from . import _lib

c_int, c_ll = ctypes.c_int, ctypes.c_longlong


def _split(idx: torch.Tensor):
    if idx.dtype == torch.int32:
        return idx, None
    if idx.dtype == torch.int64:
        return None, idx
    raise TypeError("flat indices must be int32 or int64")


def csr_pack(flat_idx: torch.Tensor, rows: int, n: int, *, narrow_cols: bool, want_order: bool, want_inverse: bool):
    """Group ``flat = row * n + col`` entries by row on the device.

    Returns ``(row_ptr int32 [rows + 1], cols int16|int32 [nnz], order int32 [nnz] | None, inverse int32 [nnz] | None)``
    with ``flat_idx[order]`` being the row-grouped stream and ``inverse`` the inverse permutation.  Entries outside the
    matrix raise ``ValueError`` (a synchronising check of one counter).
    """
    idx = flat_idx.contiguous()
    i32, i64 = _split(idx)
    dev, nnz = idx.device, idx.numel()
    scratch = torch.zeros(2 * rows + 1, dtype=torch.int32, device=dev)
    counts, cursor, bad = scratch[:rows], scratch[rows: 2 * rows], scratch[2 * rows:]
    row_ptr = torch.empty(rows + 1, dtype=torch.int32, device=dev)
    cols = torch.empty(nnz, dtype=torch.int16 if narrow_cols else torch.int32, device=dev)
    order = torch.empty(nnz, dtype=torch.int32, device=dev) if want_order else None
    inverse = torch.empty(nnz, dtype=torch.int32, device=dev) if want_inverse else None
    rc = _lib.load().sb_csr_pack(_lib.ptr(i32), _lib.ptr(i64), c_ll(nnz), c_int(rows), c_int(n), _lib.ptr(counts), _lib.ptr(cursor),
                                 _lib.ptr(row_ptr), _lib.ptr(cols if narrow_cols else None), _lib.ptr(None if narrow_cols else cols),
                                 _lib.ptr(order), _lib.ptr(inverse), _lib.ptr(bad), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_csr_pack")
    _lib.count(3)
    if int(bad.item()):
        raise ValueError("flat index outside the matrix")
    return row_ptr, cols, order, inverse


def delta_pack(flat_idx: torch.Tensor, rows: int, n: int, *, want_inverse: bool):
    """Sorted-stream encoding: ``(base int64 [1], gaps int64 [nnz - 1], inverse int32 | None, max_gap int)`` or ``None`` when a
    row holds more entries than the in-row sorter takes (the caller then sorts with the framework)."""
    dev, nnz = flat_idx.device, flat_idx.numel()
    row_ptr, cols, order, inverse = csr_pack(flat_idx, rows, n, narrow_cols=False, want_order=True, want_inverse=want_inverse)
    gaps = torch.empty(max(0, nnz - 1), dtype=torch.int64, device=dev)
    base = torch.empty(1, dtype=torch.int64, device=dev)
    stats = torch.zeros(2, dtype=torch.int64, device=dev)          # [max gap, rows left unsorted (low 32 bits)]
    rc = _lib.load().sb_delta_pack(_lib.ptr(row_ptr), c_int(rows), c_int(n), c_ll(nnz), _lib.ptr(cols), _lib.ptr(order), _lib.ptr(inverse),
                                   _lib.ptr(gaps), _lib.ptr(base), _lib.ptr(stats[0:1]), _lib.ptr(stats[1:2]), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_delta_pack")
    _lib.count(2)
    max_gap, unsorted = (int(v) for v in stats.tolist())
    if unsorted & 0xFFFFFFFF:
        return None
    return base, gaps, inverse, max_gap


def amax_sumsq(x: torch.Tensor) -> torch.Tensor:
    """``stats`` int32-typed pair on the device: ``stats[0]`` = bits of ``max |x|`` (fp32), ``stats[1]`` = bits of ``sum x^2``."""
    assert x.dtype in (torch.bfloat16, torch.float32) and x.is_contiguous()
    stats = torch.zeros(2, dtype=torch.int32, device=x.device)
    rc = _lib.load().sb_amax_sumsq(_lib.ptr(x), c_ll(x.numel()), c_int(int(x.dtype == torch.bfloat16)), _lib.ptr(stats), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_amax_sumsq")
    _lib.count(1)
    return stats


def sum_squares(x: torch.Tensor) -> torch.Tensor:
    """fp32 scalar tensor ``sum x^2`` (one pass, no host read)."""
    return amax_sumsq(x)[1:2].view(torch.float32).reshape(())


def quantize_symmetric(x: torch.Tensor, bits: int):
    """Per-tensor symmetric codes with a clamped range: int8 in ``[-127, 127]`` (``bits == 8``) or nibbles ``q + 8`` with
    ``q`` in ``[-7, 7]``, two per byte (``bits == 4``).  Returns ``(codes, scale fp32 [1])``; an all-zero tensor gets scale 1."""
    x = x.contiguous()
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    stats = amax_sumsq(x)
    n = x.numel()
    out = torch.empty(n if bits == 8 else (n + 1) // 2, dtype=torch.int8 if bits == 8 else torch.uint8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    rc = _lib.load().sb_quantize_sym(_lib.ptr(x), c_ll(n), c_int(int(x.dtype == torch.bfloat16)), c_int(bits), _lib.ptr(stats), _lib.ptr(scale),
                                     _lib.ptr(out), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_quantize_sym")
    _lib.count(1)
    return (out.view(x.shape) if bits == 8 else out), scale


def move_rows(src: torch.Tensor, index: torch.Tensor, *, scatter_into: torch.Tensor | None = None) -> torch.Tensor:
    """``src[index]`` (gather) or, with ``scatter_into``, ``scatter_into[index[i]] = src[i]`` for contiguous bf16 rows."""
    assert src.dtype == torch.bfloat16 and src.dim() == 2 and src.is_contiguous() and src.shape[1] % 8 == 0
    index = index.to(torch.int64).contiguous()
    count = index.numel()
    if scatter_into is None:
        dst = torch.empty(count, src.shape[1], dtype=src.dtype, device=src.device)
    else:
        dst = scatter_into
        assert dst.is_contiguous() and dst.dtype == src.dtype and dst.shape[1] == src.shape[1]
    rc = _lib.load().sb_move_rows(_lib.ptr(src), _lib.ptr(dst), _lib.ptr(index), c_ll(count), c_int(src.shape[1]),
                                  c_int(int(scatter_into is not None)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_move_rows")
    _lib.count(1)
    return dst


def quantize_rows_int8(x: torch.Tensor):
    """Per-row symmetric int8 codes of a ``[rows, r]`` fp32 / bf16 matrix (rows may be strided): ``(int8 [rows, r], fp32 scale [rows, 1])``."""
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype in (torch.float32, torch.bfloat16)
    rows, r = x.shape
    q = torch.empty(rows, r, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, 1, dtype=torch.float32, device=x.device)
    rc = _lib.load().sb_quantize_rows_int8(_lib.ptr(x), c_int(int(x.dtype == torch.bfloat16)), c_ll(rows), c_int(r), c_int(x.stride(0)), _lib.ptr(q),
                                           _lib.ptr(scale), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_quantize_rows_int8")
    _lib.count(1)
    return q, scale


def dequantize_rows_int8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """bf16 ``q * scale[row]`` for contiguous int8 ``[rows, r]`` codes and fp32 per-row scales."""
    rows, r = q.shape
    out = torch.empty(rows, r, dtype=torch.bfloat16, device=q.device)
    rc = _lib.load().sb_dequantize_rows_int8(_lib.ptr(q.contiguous()), _lib.ptr(scale.reshape(-1).contiguous()), c_ll(rows), c_int(r), _lib.ptr(out),
                                             _lib.stream_ptr())
    _lib.check_rc(rc, "sb_dequantize_rows_int8")
    _lib.count(1)
    return out
