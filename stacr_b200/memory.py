"""Simple byte accounting (reference: stacr/memory.py:8-82)."""

from __future__ import annotations

import math

import torch


def dtype_bytes(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def dense_bytes(shape: tuple[int, ...], dtype: torch.dtype) -> int:
    count = 1
    for d in shape:
        if isinstance(d, bool) or int(d) != d or d < 0:
            raise ValueError("Shape dimensions must be nonnegative integers")
        count *= int(d)
    return count * dtype_bytes(dtype)


def _bits_to_bytes(count: int, bits: int | None, value_bytes: int) -> int:
    return math.ceil(count * bits / 8) if bits else count * value_bytes


def stacr_stored_bytes(
    shape: tuple[int, ...],
    rank: int,
    dtype: torch.dtype = torch.float16,
    residual_budget: float = 0.005,
    index_bytes: int = 4,
    include_basis: bool = False,
    *,
    coeff_bits: int | None = None,
    residual_bits: int | None = None,
    basis_dtype: torch.dtype | None = None,
    include_scales: bool = True,
) -> int:
    """Factor payload estimate: coefficients + sparse residual (+ basis), excluding workspaces.

    ``None`` bit widths keep the activation dtype; explicit 4/8-bit storage adds a 4-byte scale;
    ``residual_bits=0`` is the unquantised sparse channel, which still stores a unit scale.
    """
    dense_bytes(shape, dtype)
    if isinstance(rank, bool) or int(rank) != rank or rank < 1:
        raise ValueError("rank must be a positive integer")
    if not math.isfinite(residual_budget) or not 0 <= residual_budget <= 1:
        raise ValueError("residual_budget must be between 0 and 1")
    if index_bytes not in (2, 4, 8):
        raise ValueError("index_bytes must be 2, 4, or 8")
    if coeff_bits not in (None, 0, 4, 8) or residual_bits not in (None, 0, 4, 8):
        raise ValueError("Bit widths must be None, 0, 4, or 8")
    if len(shape) == 0:
        return dense_bytes(shape, dtype)
    features = int(shape[-1])
    if features == 0:
        return 0
    rows = math.prod(int(d) for d in shape[:-1])
    r = min(int(rank), features)
    vb = dtype_bytes(dtype)
    n_coeff = rows * r
    total = _bits_to_bytes(n_coeff, coeff_bits, vb)
    if include_scales and coeff_bits and n_coeff:
        total += 4
    n_res = int(round(float(residual_budget) * rows * features))
    total += n_res * index_bytes + _bits_to_bytes(n_res, residual_bits, vb)
    if include_scales and residual_bits is not None and n_res:
        total += 4
    if include_basis:
        total += features * r * dtype_bytes(basis_dtype or dtype)
    return int(total)


def saved_surface_predictor(saved_bytes: float, baseline_peak_bytes: float) -> float:
    """SSP = positive replaceable saved-surface bytes divided by the baseline peak."""
    if not math.isfinite(baseline_peak_bytes) or baseline_peak_bytes <= 0:
        raise ValueError("baseline_peak_bytes must be finite and positive")
    if not math.isfinite(saved_bytes):
        raise ValueError("saved_bytes must be finite")
    return max(0.0, float(saved_bytes)) / float(baseline_peak_bytes)
