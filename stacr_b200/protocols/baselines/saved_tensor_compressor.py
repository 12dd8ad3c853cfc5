"""Saved-tensor hooks that store TT / Tucker / SVD factorisations of large saved activations (a comparator).

Parity: stacr/protocols/baselines/saved_tensor_compressor.py:16-237 of the reference project; the decompositions
come from ``stacr_b200.protocols.compression`` (no third-party tensor library is needed).
"""

from __future__ import annotations

import math
import time
from contextlib import contextmanager
from typing import Any, Dict, Tuple

import torch

from ..compression import Compressor


class SavedTensorCompressor:
    def __init__(self, method: str = "tt", rank: int = 8, min_numel: int = 1 << 16, quantize_bits: int | None = None):
        if method not in ("tt", "tucker", "svd"):
            raise ValueError("method must be tt, tucker or svd")
        self.method, self.rank, self.min_numel, self.bits = method, int(rank), int(min_numel), quantize_bits
        self.reset()

    def reset(self) -> None:
        self.packed = self.skipped = 0
        self.raw_bytes = self.stored_bytes = 0
        self.pack_seconds = self.unpack_seconds = 0.0

    def _tensorize_shape(self, numel: int) -> Tuple[int, ...]:
        """Factor ``numel`` into up to four near-equal dimensions."""
        dims, rest = [], numel
        for k in (4, 3, 2):
            target = round(rest ** (1.0 / k))
            d = next((c for c in range(max(2, target), 1, -1) if rest % c == 0), None)
            if d is None:
                continue
            dims.append(d)
            rest //= d
        dims.append(rest)
        return tuple(sorted(d for d in dims if d > 1)) or (numel,)

    def _normalize_tucker_rank(self, shape):
        return tuple(max(1, min(self.rank, d)) for d in shape)

    def pack(self, tensor: torch.Tensor):
        keep = (not tensor.is_floating_point() or tensor.numel() < self.min_numel or (tensor.requires_grad and tensor.is_leaf) or tensor.dim() < 2)
        if keep:
            self.skipped += 1
            return ("raw", tensor)
        t0 = time.perf_counter()
        flat = tensor.detach().reshape(tensor.shape[0], -1) if self.method == "svd" else tensor.detach().reshape(-1)
        if self.method == "svd":
            factors = Compressor.compress_svd_factors(flat, self.rank, use_lowrank=True)
        else:
            shape = self._tensorize_shape(tensor.numel())
            flat2 = flat.reshape(shape[0], -1)
            factors = (Compressor.compress_tt_factors(flat2, shape, self.rank) if self.method == "tt"
                       else Compressor.compress_tucker_factors(flat2, shape, self._normalize_tucker_rank(shape)))
        self.pack_seconds += time.perf_counter() - t0
        self.packed += 1
        self.raw_bytes += tensor.numel() * tensor.element_size()
        self.stored_bytes += Compressor.get_memory_usage(factors)
        return (self.method, factors, tuple(tensor.shape), tensor.dtype)

    def unpack(self, packed):
        if packed[0] == "raw":
            return packed[1]
        t0 = time.perf_counter()
        method, factors, shape, dtype = packed
        out = {"svd": Compressor.decompress_svd, "tt": Compressor.decompress_tt, "tucker": Compressor.decompress_tucker}[method](factors)
        self.unpack_seconds += time.perf_counter() - t0
        return out.reshape(shape).to(dtype)

    @contextmanager
    def context(self):
        with torch.autograd.graph.saved_tensors_hooks(self.pack, self.unpack):
            yield self

    def get_stats(self) -> Dict[str, Any]:
        return {"method": self.method, "rank": self.rank, "packed": self.packed, "skipped": self.skipped, "raw_bytes": self.raw_bytes,
                "stored_bytes": self.stored_bytes, "ratio": self.raw_bytes / self.stored_bytes if self.stored_bytes else None,
                "pack_seconds": self.pack_seconds, "unpack_seconds": self.unpack_seconds}
