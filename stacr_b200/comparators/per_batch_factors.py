"""Per-batch factorisation baselines on a single activation tensor (parity: comparators/per_batch_factors.py)."""

from __future__ import annotations

import math
import time
from typing import Any

import torch

from ..protocols.compression import Compressor


def svd_reconstruct(tensor: torch.Tensor, rank: int) -> torch.Tensor:
    flat = tensor.reshape(-1, tensor.shape[-1])
    return Compressor.decompress_svd(Compressor.compress_svd_factors(flat, rank)).reshape(tensor.shape).to(tensor.dtype)


def _square_shape(flat: torch.Tensor):
    def two(n):
        a = int(math.isqrt(n))
        while a > 1 and n % a:
            a -= 1
        return (a, n // a)
    return two(flat.shape[0]) + two(flat.shape[1])


def tucker_like_reconstruct(tensor: torch.Tensor, rank: int) -> torch.Tensor:
    flat = tensor.reshape(-1, tensor.shape[-1])
    shape = _square_shape(flat)
    data = Compressor.compress_tucker_factors(flat, shape, [min(rank, d) for d in shape])
    return Compressor.decompress_tucker(data).reshape(tensor.shape).to(tensor.dtype)


def tt_like_reconstruct(tensor: torch.Tensor, rank: int) -> torch.Tensor:
    flat = tensor.reshape(-1, tensor.shape[-1])
    return Compressor.decompress_tt(Compressor.compress_tt_factors(flat, _square_shape(flat), rank)).reshape(tensor.shape).to(tensor.dtype)


def factorization_benchmark(tensor: torch.Tensor, rank: int = 8) -> list[dict[str, Any]]:
    rows = []
    for name, fn in (("svd", svd_reconstruct), ("tucker", tucker_like_reconstruct), ("tt", tt_like_reconstruct)):
        t0 = time.perf_counter()
        rec = fn(tensor, rank)
        rows.append({"method": name, "rank": rank, "seconds": time.perf_counter() - t0,
                     "relative_error": float((rec.float() - tensor.float()).norm() / tensor.float().norm().clamp_min(1e-30))})
    return rows
