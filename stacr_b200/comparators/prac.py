"""PRAC-style comparator as a stand-alone compressor: a fixed Gaussian subspace that is never tracked.

Parity: comparators/prac.py (``PRACConfig``, ``PRACCompressor.projection/reconstruct``).  The layer form of
the same method (used inside a training run) is ``stacr_b200.comparators.activation.PracLinear``; this class is
the tensor-in/tensor-out form the mechanism-replay script compares against ``STACRCompressor``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class PRACConfig:
    rank: int = 8
    seed: int = 0


class PRACCompressor:
    """Projects the last dimension on ``rank`` random directions drawn once per feature width.

    The directions are N(0, 1/rank) entries from a CPU generator seeded by ``seed + features`` so that every
    device sees the same subspace; they are not orthonormalised and never updated, which is the point of the
    comparison with a tracked basis.
    """

    def __init__(self, config: PRACConfig | None = None):
        self.config = config if config is not None else PRACConfig()
        self._cache: dict = {}

    def projection(self, features: int, device, dtype) -> torch.Tensor:
        features = int(features)
        device = torch.device(device)
        slot = (features, device)
        p = self._cache.get(slot)
        if p is None:
            r = min(max(int(self.config.rank), 1), features)
            g = torch.Generator().manual_seed(int(self.config.seed) + features)
            p = (torch.randn(features, r, generator=g) * r ** -0.5).to(device)
            self._cache[slot] = p
        return p.to(dtype)

    def compress(self, tensor: torch.Tensor) -> torch.Tensor:
        """Coefficients ``[rows, rank]`` of ``tensor`` flattened to ``[rows, features]``."""
        flat = tensor.reshape(-1, tensor.shape[-1])
        return flat @ self.projection(flat.shape[-1], tensor.device, tensor.dtype)

    def reconstruct(self, tensor: torch.Tensor) -> torch.Tensor:
        p = self.projection(tensor.shape[-1], tensor.device, tensor.dtype)
        return (self.compress(tensor) @ p.t()).reshape(tensor.shape)

    def stored_bytes(self, tensor: torch.Tensor) -> int:
        """Bytes kept for backward: the coefficients only (the subspace is regenerated from the seed)."""
        rows = tensor.numel() // tensor.shape[-1]
        return rows * min(max(int(self.config.rank), 1), tensor.shape[-1]) * tensor.element_size()
