"""Storage-only path: compress arbitrary saved tensors through ``saved_tensors_hooks``.

``unpack`` must hand autograd a dense tensor, so this path rebuilds the activation in backward
and cannot express the factor-native weight gradient; it exists for reconstruction telemetry
and for graphs not built from linear modules.  The measured method is ``apply_stacr``.
Parity: stacr/compressor.py:13-140 of the reference project.
"""

from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any

import torch

from .oja import OjaBasis
from .residual import SparseResidual, select_topk_residual


@dataclass
class STACRConfig:
    rank: int = 8
    residual_budget: float = 0.005
    min_features: int = 128
    min_numel: int = 4096
    oja_lr: float = 0.01
    update_interval: int = 1
    warmup_steps: int = 0
    residual_mode: str = "topk"
    post_warmup_mode: str = "full"
    turbo_after_step: int | None = None
    basis_dtype: str = "float32"


@dataclass
class PackedActivation:
    shape: tuple[int, ...]
    dtype: torch.dtype
    coeff: torch.Tensor
    basis: torch.Tensor
    residual: SparseResidual | None


def _resolve_basis_dtype(spec: str, activation_dtype: torch.dtype) -> torch.dtype:
    key = str(spec).lower()
    if key in ("auto", "activation"):
        return activation_dtype
    return {"float16": torch.float16, "fp16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16,
            "bf16": torch.bfloat16}.get(key, torch.float32)


class STACRCompressor:
    """Pack/unpack hooks with one persistent Oja basis per (feature size, device)."""

    def __init__(self, config: STACRConfig | None = None):
        self.config = config or STACRConfig()
        self.step = 0
        self._bases: dict[tuple[int, torch.device], OjaBasis] = {}

    def set_step(self, step: int) -> None:
        self.step = int(step)

    def advance(self) -> None:
        self.step += 1

    def _basis_for(self, t: torch.Tensor) -> OjaBasis:
        key = (int(t.shape[-1]), t.device)
        state = self._bases.get(key)
        if state is None:
            state = OjaBasis(key[0], self.config.rank, dtype=_resolve_basis_dtype(self.config.basis_dtype, t.dtype), device=t.device)
            self._bases[key] = state
        return state

    @staticmethod
    def is_parameter(t: torch.Tensor) -> bool:
        """Weights and biases (and views of them, e.g. the transposed weight autograd saves)."""
        if isinstance(t, torch.nn.Parameter) or (t.requires_grad and t.is_leaf):
            return True
        base = getattr(t, "_base", None)
        return base is not None and STACRCompressor.is_parameter(base)

    def should_compress(self, t: torch.Tensor) -> bool:
        c = self.config
        return (
            t.is_floating_point() and t.dim() >= 2 and not self.is_parameter(t)
            and int(t.shape[-1]) >= int(c.min_features) and t.numel() >= int(c.min_numel)
        )

    def _residual_on(self) -> bool:
        c = self.config
        if c.turbo_after_step is not None and self.step >= int(c.turbo_after_step):
            return False
        return c.residual_mode != "none"

    def pack(self, t: torch.Tensor) -> Any:
        c = self.config
        if not self.should_compress(t) or self.step < int(c.warmup_steps):
            return t
        x = t.detach()
        flat = x.reshape(-1, x.shape[-1])
        state = self._basis_for(x)
        if self.step % max(1, int(c.update_interval)) == 0:
            state.update(flat, lr=float(c.oja_lr))
        q = state.shared(dtype=x.dtype)
        coeff = (flat @ q).to(x.dtype)
        residual = None
        if self._residual_on():
            residual = select_topk_residual(x - (coeff @ q.t()).reshape_as(x), float(c.residual_budget))
        return PackedActivation(tuple(x.shape), x.dtype, coeff, q, residual)

    def unpack(self, packed: Any) -> torch.Tensor:
        if not isinstance(packed, PackedActivation):
            return packed
        dense = (packed.coeff @ packed.basis.t()).reshape(packed.shape)
        if packed.residual is not None:
            dense = dense + packed.residual.dense(device=dense.device, dtype=dense.dtype)
        return dense.to(packed.dtype)


@contextmanager
def stacr_saved_tensors(compressor: STACRCompressor):
    """Run a forward with the compressor installed as saved-tensor hooks."""
    with torch.autograd.graph.saved_tensors_hooks(compressor.pack, compressor.unpack):
        yield compressor
