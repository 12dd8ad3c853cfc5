"""Byte estimates for one compressed activation, as an itemised ledger.

``payload_ledger`` lists what a wrapped layer keeps for backward, channel by channel (coefficients, residual indices, residual
values, quantisation scales, optionally the basis); ``stacr_stored_bytes`` is its total and ``saved_surface_predictor`` the share
of a baseline peak that a replaceable saved surface accounts for.  Workspaces are not part of the estimate.

API parity: stacr/memory.py:8-82 of the reference project (same signatures, defaults, rounding and error conditions).
"""

from __future__ import annotations

import math
from typing import NamedTuple

import torch

_ALLOWED_BITS = (None, 0, 4, 8)
_SCALE_BYTES = 4  # one fp32 scale per quantised channel


def dtype_bytes(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def _whole_number(value, *, at_least: int) -> bool:
    return not isinstance(value, bool) and int(value) == value and value >= at_least


def dense_bytes(shape: tuple[int, ...], dtype: torch.dtype) -> int:
    if not all(_whole_number(d, at_least=0) for d in shape):
        raise ValueError("Shape dimensions must be nonnegative integers")
    return math.prod(int(d) for d in shape) * dtype_bytes(dtype)


class Ledger(NamedTuple):
    """Bytes per stored channel of one activation."""

    coefficients: int = 0
    residual_indices: int = 0
    residual_values: int = 0
    scales: int = 0
    basis: int = 0

    @property
    def total(self) -> int:
        return int(sum(self))


def _channel_bytes(entries: int, bits: int | None, element_bytes: int) -> int:
    """``entries`` values at ``bits`` each, packed; ``None`` / 0 bits mean the activation's own element size."""
    return entries * element_bytes if not bits else math.ceil(entries * bits / 8)


def payload_ledger(shape, rank, dtype=torch.float16, residual_budget=0.005, index_bytes=4, include_basis=False, *,
                   coeff_bits=None, residual_bits=None, basis_dtype=None, include_scales=True) -> Ledger:
    """Validate the arguments and itemise the payload of an activation of ``shape`` (last dimension = features)."""
    dense = dense_bytes(shape, dtype)
    problems = (
        (not _whole_number(rank, at_least=1), "rank must be a positive integer"),
        (not (math.isfinite(residual_budget) and 0 <= residual_budget <= 1), "residual_budget must be between 0 and 1"),
        (index_bytes not in (2, 4, 8), "index_bytes must be 2, 4, or 8"),
        (coeff_bits not in _ALLOWED_BITS or residual_bits not in _ALLOWED_BITS, "Bit widths must be None, 0, 4, or 8"),
    )
    for failed, message in problems:
        if failed:
            raise ValueError(message)
    if len(shape) == 0:
        return Ledger(coefficients=dense)     # a scalar is kept as it is
    features = int(shape[-1])
    if features == 0:
        return Ledger()
    element = dtype_bytes(dtype)
    rows = math.prod(int(d) for d in shape[:-1])
    kept_rank = min(int(rank), features)
    n_coeff = rows * kept_rank
    n_residual = int(round(float(residual_budget) * rows * features))
    # a scale accompanies explicitly quantised coefficients, and every residual channel whose width was stated (0 = unquantised
    # values with a unit scale)
    scaled_channels = int(bool(coeff_bits) and n_coeff > 0) + int(residual_bits is not None and n_residual > 0)
    return Ledger(
        coefficients=_channel_bytes(n_coeff, coeff_bits, element),
        residual_indices=n_residual * index_bytes,
        residual_values=_channel_bytes(n_residual, residual_bits, element),
        scales=_SCALE_BYTES * scaled_channels if include_scales else 0,
        basis=features * kept_rank * dtype_bytes(basis_dtype or dtype) if include_basis else 0,
    )


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
    """Total of ``payload_ledger``: coefficients + sparse residual (+ scales, + basis when asked for)."""
    return payload_ledger(shape, rank, dtype, residual_budget, index_bytes, include_basis, coeff_bits=coeff_bits,
                          residual_bits=residual_bits, basis_dtype=basis_dtype, include_scales=include_scales).total


def saved_surface_predictor(saved_bytes: float, baseline_peak_bytes: float) -> float:
    """SSP: the replaceable saved-surface bytes (negative counts as none) as a fraction of the baseline peak."""
    peak_ok = math.isfinite(baseline_peak_bytes) and baseline_peak_bytes > 0
    if not peak_ok or not math.isfinite(saved_bytes):
        raise ValueError("saved_bytes must be finite" if peak_ok else "baseline_peak_bytes must be finite and positive")
    return max(float(saved_bytes), 0.0) / float(baseline_peak_bytes)
