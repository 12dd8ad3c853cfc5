"""Compact encodings for the flat indices of the sparse residual.

A residual entry is addressed by ``flat = row * N + col``.  Two lossless encodings shrink the
index stream: **CSR** (row pointers plus narrow column ids, int16 when ``N < 32768``) and
**delta** (sorted indices stored as first value plus narrow gaps).  Both can carry the inverse
permutation so the original entry order (which the value stream follows) is restorable.
API parity: stacr/index_compression.py:43-974 of the reference project.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from enum import Enum
from typing import Any, Dict, Optional, Union

import torch


class IndexCompressionMode(Enum):
    NONE = "none"
    CSR = "csr"
    DELTA = "delta"


def _nbytes(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.numel() * t.element_size()


def _dtype_bytes(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def _choose_col_dtype(N: int) -> torch.dtype:
    if N < 32768:
        return torch.int16
    return torch.int32 if N <= 2**31 else torch.int64


def _narrowest_signed(max_value: int) -> torch.dtype:
    if max_value <= 32767:
        return torch.int16
    return torch.int32 if max_value < 2**31 else torch.int64


@dataclass
class CompressedIndices:
    """Encoded index stream.  In delta mode ``col_indices`` holds the gaps and ``delta_base`` the first index."""

    mode: IndexCompressionMode
    row_ptrs: Optional[torch.Tensor] = None
    col_indices: Optional[torch.Tensor] = None
    delta_base: Optional[torch.Tensor] = None
    sort_indices: Optional[torch.Tensor] = None
    nnz: int = 0
    B_flat: int = 0
    N: int = 0
    original_dtype: torch.dtype = torch.int32

    def _tensors(self):
        return (self.row_ptrs, self.col_indices, self.delta_base, self.sort_indices)

    def memory_bytes(self) -> int:
        return sum(_nbytes(t) for t in self._tensors())

    def to(self, device) -> "CompressedIndices":
        move = lambda t: None if t is None else t.to(device)
        return CompressedIndices(
            self.mode, move(self.row_ptrs), move(self.col_indices), move(self.delta_base), move(self.sort_indices),
            self.nnz, self.B_flat, self.N, self.original_dtype,
        )


def compress_indices(
    flat_indices: torch.Tensor,
    B_flat: int,
    N: int,
    mode: Union[str, IndexCompressionMode] = "csr",
    preserve_order: bool = True,
) -> CompressedIndices:
    """Encode ``flat_indices`` (``row * N + col``) of a ``B_flat x N`` matrix."""
    mode = IndexCompressionMode(mode) if isinstance(mode, str) else mode
    nnz = int(flat_indices.numel())
    meta = dict(nnz=nnz, B_flat=int(B_flat), N=int(N), original_dtype=flat_indices.dtype)
    dev = flat_indices.device
    if nnz == 0:
        empty = torch.empty(0, dtype=flat_indices.dtype, device=dev)
        rp = torch.zeros(B_flat + 1, dtype=torch.int32, device=dev) if mode is IndexCompressionMode.CSR else None
        return CompressedIndices(mode, row_ptrs=rp, col_indices=empty, **meta)
    if mode is IndexCompressionMode.NONE:
        return CompressedIndices(mode, col_indices=flat_indices, **meta)
    if flat_indices.is_cuda and flat_indices.dtype in (torch.int32, torch.int64) and nnz < 2**31 - 1 and B_flat < 2**31 - 1 and N < 2**31 - 1:
        packed = _compress_on_device(flat_indices, B_flat, N, mode, preserve_order, meta)
        if packed is not None:
            return packed
    wide = flat_indices.long()
    if mode is IndexCompressionMode.CSR:
        rows = torch.div(wide, N, rounding_mode="floor")
        cols = wide - rows * N
        order = torch.argsort(rows, stable=True)
        counts = torch.bincount(rows, minlength=B_flat)
        ptr = torch.zeros(B_flat + 1, dtype=torch.int32 if nnz < 2**31 else torch.int64, device=dev)
        ptr[1:] = torch.cumsum(counts, 0)
        inverse = torch.argsort(order) if preserve_order else None
        return CompressedIndices(mode, row_ptrs=ptr, col_indices=cols[order].to(_choose_col_dtype(N)), sort_indices=inverse, **meta)
    if mode is IndexCompressionMode.DELTA:
        ordered, order = torch.sort(wide)
        base = ordered[:1].to(torch.int32 if B_flat * N <= 2**31 else torch.int64)
        if nnz > 1:
            gaps = ordered[1:] - ordered[:-1]
            gaps = gaps.to(_narrowest_signed(int(gaps.max())))
        else:
            gaps = torch.empty(0, dtype=torch.int16, device=dev)
        inverse = torch.argsort(order) if preserve_order else None
        return CompressedIndices(mode, col_indices=gaps, delta_base=base, sort_indices=inverse, **meta)
    raise ValueError(f"Unknown compression mode: {mode}")


def _compress_on_device(flat_indices, B_flat, N, mode, preserve_order, meta):
    """The same encodings produced by the counting-sort / in-row-sort kernels (``ops/csrc/index_pack.cu``): no library sort,
    no ``bincount``/``cumsum`` chain.  The order inside a CSR row is the scatter's, not the input's; the inverse permutation
    that comes with it restores the original order exactly as the framework path's does.  ``None`` = not handled here."""
    from .ops import pack_ops

    if mode is IndexCompressionMode.CSR:
        row_ptr, cols, _, inverse = pack_ops.csr_pack(flat_indices, B_flat, N, narrow_cols=N < 32768, want_order=False, want_inverse=preserve_order)
        return CompressedIndices(mode, row_ptrs=row_ptr, col_indices=cols, sort_indices=None if inverse is None else inverse.long(), **meta)
    if mode is IndexCompressionMode.DELTA:
        out = pack_ops.delta_pack(flat_indices, B_flat, N, want_inverse=preserve_order)
        if out is None:
            return None
        base, gaps, inverse, max_gap = out
        base = base.to(torch.int32 if B_flat * N <= 2**31 else torch.int64)
        gaps = gaps.to(_narrowest_signed(max_gap)) if gaps.numel() else torch.empty(0, dtype=torch.int16, device=flat_indices.device)
        return CompressedIndices(mode, col_indices=gaps, delta_base=base, sort_indices=None if inverse is None else inverse.long(), **meta)
    return None


def decompress_indices(compressed: CompressedIndices, restore_order: bool = True) -> torch.Tensor:
    """Inverse of :func:`compress_indices`."""
    c = compressed
    anchor = c.col_indices if c.col_indices is not None else c.delta_base
    dev = anchor.device if anchor is not None else torch.device("cpu")
    if c.nnz == 0:
        return torch.empty(0, dtype=c.original_dtype, device=dev)
    if c.mode is IndexCompressionMode.NONE:
        return c.col_indices
    if c.mode is IndexCompressionMode.CSR:
        if c.row_ptrs is None or c.row_ptrs.numel() != c.B_flat + 1 or int(c.row_ptrs[-1]) != c.nnz:
            raise ValueError("Inconsistent CSR row pointers")
        counts = (c.row_ptrs[1:] - c.row_ptrs[:-1]).long()
        rows = torch.repeat_interleave(torch.arange(c.B_flat, device=dev), counts)
        flat = rows * c.N + c.col_indices.long()
    elif c.mode is IndexCompressionMode.DELTA:
        flat = torch.cat((c.delta_base.long(), c.col_indices.long())).cumsum(0)
    else:
        raise ValueError(f"Unknown compression mode: {c.mode}")
    if restore_order and c.sort_indices is not None:
        flat = flat[c.sort_indices]
    return flat.to(c.original_dtype)


def estimate_index_compression(
    B_flat: int,
    N: int,
    nnz: int,
    mode: Union[str, IndexCompressionMode] = "csr",
    original_dtype: torch.dtype = torch.int32,
    preserve_order: bool = True,
) -> Dict[str, Any]:
    """Predicted bytes of an encoding from shapes alone (delta assumes 16-bit gaps)."""
    mode = IndexCompressionMode(mode) if isinstance(mode, str) else mode
    original = nnz * _dtype_bytes(original_dtype)
    order_bytes = nnz * 4 if preserve_order else 0
    if mode is IndexCompressionMode.CSR:
        packed = (B_flat + 1) * 4 + nnz * (2 if N < 32768 else 4) + order_bytes
    elif mode is IndexCompressionMode.DELTA:
        packed = 4 + max(0, nnz - 1) * 2 + order_bytes
    else:
        packed = original
    return {
        "original_bytes": original,
        "compressed_bytes": packed,
        "compression_ratio": original / packed if packed > 0 else float("inf"),
        "savings_percent": (1 - packed / original) * 100 if original > 0 else 0,
        "savings_bytes": original - packed,
        "mode": mode.value,
        "B_flat": B_flat,
        "N": N,
        "nnz": nnz,
    }


def csr_memory_savings(
    batch_size: int, features: int, nnz: int, dtype: torch.dtype = torch.float32, index_dtype: torch.dtype = torch.int32
) -> Dict[str, float]:
    """Bytes of a CSR matrix (pointers + columns + values) against the dense matrix."""
    vb, ib = _dtype_bytes(dtype), _dtype_bytes(index_dtype)
    dense = batch_size * features * vb
    crow, col, values = (batch_size + 1) * ib, nnz * ib, nnz * vb
    csr = crow + col + values
    cells = batch_size * features
    return {
        "dense_bytes": dense,
        "csr_bytes": csr,
        "crow_bytes": crow,
        "col_bytes": col,
        "values_bytes": values,
        "savings_bytes": dense - csr,
        "sparsity": 1.0 - nnz / cells if cells > 0 else 0.0,
        "compression_ratio": dense / csr if csr > 0 else float("inf"),
    }


def compress_activation_to_csr(activation: torch.Tensor, threshold: float = 0.0, index_dtype: torch.dtype = torch.int32) -> torch.Tensor:
    """Sparse-CSR tensor of the entries with ``|a| > threshold``."""
    if activation.ndim != 2:
        raise ValueError(f"Expected 2D tensor, got shape {activation.shape}")
    rows, cols = activation.shape
    keep = activation.abs() > threshold
    r, c = keep.nonzero(as_tuple=True)
    crow = torch.zeros(rows + 1, dtype=index_dtype, device=activation.device)
    crow[1:] = torch.cumsum(torch.bincount(r, minlength=rows), 0).to(index_dtype)
    return torch.sparse_csr_tensor(crow, c.to(index_dtype), activation[keep], size=(rows, cols), dtype=activation.dtype, device=activation.device)


def _varint_bits(gap: int) -> int:
    return 8 if gap < 128 else 16 if gap < 16384 else 32


def analyze_delta_compression_potential(indices: torch.Tensor) -> Dict[str, float]:
    """Gap statistics of a sorted index stream and the size of a 1/2/4-byte variable-length coding."""
    n = int(indices.numel())
    if n < 2:
        return {
            "num_indices": n, "avg_delta": 0.0, "max_delta": 0, "min_delta": 0, "original_bytes": n * 4, "delta_bytes": n * 4,
            "compression_ratio": 1.0, "delta_histogram": {"< 128 (1 byte)": 0, "128-16383 (2 bytes)": 0, ">= 16384 (4 bytes)": 0},
        }
    gaps = (indices[1:].long() - indices[:-1].long())
    small = int((gaps < 128).sum())
    medium = int(((gaps >= 128) & (gaps < 16384)).sum())
    large = int((gaps >= 16384).sum())
    bits_delta = 32 + small * 8 + medium * 16 + large * 32
    bits_orig = n * 32
    return {
        "num_indices": n,
        "avg_delta": float(gaps.float().mean()),
        "max_delta": int(gaps.max()),
        "min_delta": int(gaps.min()),
        "original_bytes": bits_orig // 8,
        "delta_bytes": bits_delta // 8,
        "compression_ratio": bits_orig / bits_delta if bits_delta else float("inf"),
        "delta_histogram": {"< 128 (1 byte)": small, "128-16383 (2 bytes)": medium, ">= 16384 (4 bytes)": large},
    }


class DeltaEncodedIndices:
    """Sorted indices kept as first value + gaps in the narrowest signed dtype that fits."""

    def __init__(self, indices: torch.Tensor, dtype: torch.dtype = torch.int32):
        self.dtype = dtype
        self.num_indices = int(indices.numel())
        ordered = torch.sort(indices.long()).values
        if self.num_indices == 0:
            self.base = torch.zeros(1, dtype=dtype, device=indices.device)
            self.deltas = torch.empty(0, dtype=torch.int16, device=indices.device)
            return
        self.base = ordered[:1].to(dtype)
        gaps = ordered[1:] - ordered[:-1]
        width = _narrowest_signed(int(gaps.max())) if gaps.numel() else torch.int16
        self.deltas = gaps.to(width)

    def decode(self) -> torch.Tensor:
        if self.num_indices == 0:
            return torch.empty(0, dtype=self.dtype, device=self.base.device)
        return torch.cat((self.base.long(), self.deltas.long())).cumsum(0).to(self.dtype)

    def memory_bytes(self) -> int:
        return _nbytes(self.base) + _nbytes(self.deltas)

    def __repr__(self) -> str:
        return f"DeltaEncodedIndices(n={self.num_indices}, delta_dtype={self.deltas.dtype}, bytes={self.memory_bytes()})"


class BlockOffsetEncoding:
    """Block-sparse tensor as (block id, in-block offset byte, value) triples."""

    def __init__(self, tensor: torch.Tensor, block_size: int):
        if block_size < 1 or block_size > 256:
            raise ValueError("block_size must be in [1, 256]")
        self.shape = tuple(tensor.shape)
        self.dtype = tensor.dtype
        self.block_size = int(block_size)
        flat = tensor.reshape(-1)
        self.numel = int(flat.numel())
        hits = flat.nonzero(as_tuple=True)[0]
        self.values = flat[hits].clone()
        self.offsets = (hits % self.block_size).to(torch.uint8)
        blocks = torch.div(hits, self.block_size, rounding_mode="floor")
        self.block_ids = blocks.to(torch.int32 if self.numel // self.block_size < 2**31 else torch.int64)

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(self.numel, dtype=self.dtype, device=self.values.device)
        out[self.block_ids.long() * self.block_size + self.offsets.long()] = self.values
        return out.reshape(self.shape)

    def memory_bytes(self) -> int:
        return _nbytes(self.values) + _nbytes(self.offsets) + _nbytes(self.block_ids)

    def compression_ratio(self) -> float:
        dense = self.numel * _dtype_bytes(self.dtype)
        mine = self.memory_bytes()
        return dense / mine if mine else float("inf")

    def __repr__(self) -> str:
        return f"BlockOffsetEncoding(shape={self.shape}, nnz={self.values.numel()}, block={self.block_size}, ratio={self.compression_ratio():.2f})"


class IndexCompressionStats:
    """Running totals over many encode/decode operations."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.total_indices = 0
        self.total_bytes_original = 0
        self.total_bytes_compressed = 0
        self.reconstruction_times: list[float] = []

    def record(self, indices: torch.Tensor, compressed_bytes: int, reconstruction_time: float):
        self.total_indices += int(indices.numel())
        self.total_bytes_original += _nbytes(indices)
        self.total_bytes_compressed += int(compressed_bytes)
        self.reconstruction_times.append(float(reconstruction_time))

    def average_compression_ratio(self) -> float:
        return self.total_bytes_original / self.total_bytes_compressed if self.total_bytes_compressed else 1.0

    def average_reconstruction_time(self) -> float:
        t = self.reconstruction_times
        return 1000.0 * sum(t) / len(t) if t else 0.0

    def report(self) -> Dict[str, float]:
        stats = {
            "total_indices": self.total_indices,
            "original_KB": self.total_bytes_original / 1024,
            "compressed_KB": self.total_bytes_compressed / 1024,
            "avg_compression_ratio": self.average_compression_ratio(),
            "avg_reconstruction_ms": self.average_reconstruction_time(),
            "num_operations": len(self.reconstruction_times),
        }
        print("\nIndex Compression Summary:")
        for key, value in stats.items():
            print(f"  {key}: {value:,.3f}" if isinstance(value, float) else f"  {key}: {value:,}")
        return stats


def timed_roundtrip(indices: torch.Tensor, B_flat: int, N: int, mode: str, stats: IndexCompressionStats | None = None) -> CompressedIndices:
    """Encode, time the decode, and optionally record both in ``stats``."""
    packed = compress_indices(indices, B_flat, N, mode)
    t0 = time.perf_counter()
    decompress_indices(packed)
    if stats is not None:
        stats.record(indices, packed.memory_bytes(), time.perf_counter() - t0)
    return packed


def index_dtype_recommendation(max_index: int, target: str = "memory") -> torch.dtype:
    """Narrowest dtype holding ``max_index`` (``target='memory'``) or int32 (``'speed'``)."""
    if target != "memory":
        return torch.int32
    if max_index <= 127:
        return torch.int8
    return torch.int16 if max_index <= 32767 else torch.int32


def should_use_delta_encoding(indices: torch.Tensor, threshold_ratio: float = 1.5) -> bool:
    """True when variable-length gap coding pays: ratio above threshold, or most gaps fit one byte."""
    info = analyze_delta_compression_potential(indices)
    if info["compression_ratio"] >= threshold_ratio or info["avg_delta"] < 128:
        return True
    n = len(indices)
    return n > 0 and info["delta_histogram"]["< 128 (1 byte)"] / n > 0.8
