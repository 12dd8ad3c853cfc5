"""Top-k residual container for the storage-only hook path (reference: stacr/residual.py:8-34)."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class SparseResidual:
    shape: tuple[int, ...]
    indices: torch.Tensor
    values: torch.Tensor

    def dense(self, *, device, dtype: torch.dtype) -> torch.Tensor:
        out = torch.zeros(self.shape, device=device, dtype=dtype)
        if self.indices.numel():
            out.view(-1).index_put_(
                (self.indices.to(device=device, dtype=torch.long),),
                self.values.to(device=device, dtype=dtype),
            )
        return out


def select_topk_residual(residual: torch.Tensor, budget: float) -> SparseResidual:
    """Largest-magnitude entries under a fractional budget (at least one when budget > 0)."""
    r = residual.detach()
    flat = r.reshape(-1)
    if budget <= 0 or flat.numel() == 0:
        return SparseResidual(
            tuple(r.shape),
            torch.empty(0, dtype=torch.long, device=r.device),
            torch.empty(0, dtype=r.dtype, device=r.device),
        )
    k = min(flat.numel(), max(1, int(round(float(budget) * flat.numel()))))
    idx = flat.abs().topk(k, sorted=False).indices
    return SparseResidual(tuple(r.shape), idx.long(), flat[idx].clone())
