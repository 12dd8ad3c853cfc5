"""Storage-only path: any saved activation goes through ``saved_tensors_hooks`` as rank-r coefficients + a sparse residual.

Autograd wants a dense tensor back from ``unpack``, so this path rebuilds the activation in backward and cannot express the
factor-native weight gradient; it serves reconstruction telemetry and graphs that are not made of linear modules.  The measured
method is ``apply_stacr``.

Two codecs do the arithmetic behind one ``STACRCompressor``:

* ``_KernelCodec`` (bf16 CUDA activations whose width is a multiple of 8, rank <= 32): projection on the skinny tcgen05 GEMM, exact
  global top-k of ``X - C Q^T`` by the selection kernels (the dense residual is never formed), and ``unpack`` as one rebuild kernel
  writing ``bf16(C Q^T + S)``;
* ``_FrameworkCodec`` (everything else, and the oracle of the tests): the same arithmetic in framework ops.

API parity: stacr/compressor.py:13-140 of the reference project (``STACRConfig`` fields and defaults, ``PackedActivation``,
``STACRCompressor.pack/unpack/should_compress/is_parameter/set_step/advance``, ``stacr_saved_tensors``).
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
    """What replaces a saved activation.  ``residual`` is a ``SparseResidual`` (framework codec), the selection kernels'
    ``(indices, values, scale, bits, count)`` tuple (kernel codec) or ``None``."""

    shape: tuple[int, ...]
    dtype: torch.dtype
    coeff: torch.Tensor
    basis: torch.Tensor
    residual: Any
    codec: str = "framework"


_HALF_NAMES = {"float16": torch.float16, "fp16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def _resolve_basis_dtype(spec: str, activation_dtype: torch.dtype) -> torch.dtype:
    """``auto`` / ``activation`` follow the activation; a half-precision name selects it; anything else keeps fp32."""
    name = str(spec).lower()
    return activation_dtype if name in ("auto", "activation") else _HALF_NAMES.get(name, torch.float32)


class _FrameworkCodec:
    name = "framework"

    @staticmethod
    def encode(x: torch.Tensor, rows: torch.Tensor, tracker: OjaBasis, budget: float | None) -> PackedActivation:
        q = tracker.shared(dtype=x.dtype)
        coeff = (rows @ q).to(x.dtype)
        sparse = None
        if budget is not None:
            sparse = select_topk_residual(x - (coeff @ q.t()).reshape_as(x), budget)
        return PackedActivation(tuple(x.shape), x.dtype, coeff, q, sparse)

    @staticmethod
    def decode(p: PackedActivation) -> torch.Tensor:
        dense = (p.coeff @ p.basis.t()).reshape(p.shape)
        if p.residual is not None:
            dense = dense + p.residual.dense(device=dense.device, dtype=dense.dtype)
        return dense.to(p.dtype)


class _KernelCodec:
    name = "kernels"

    @staticmethod
    def accepts(x: torch.Tensor, rank: int) -> bool:
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and 1 <= rank <= 32):
            return False
        from .ops import _lib

        return _lib.available()

    @staticmethod
    def encode(x: torch.Tensor, rows: torch.Tensor, tracker: OjaBasis, budget: float | None) -> PackedActivation:
        from .layers import _basis_views, _select_residual_kernels
        from .ops import stacr_ops

        rows = rows.contiguous()
        if rows.data_ptr() % 16:
            rows = rows.clone()                               # the kernels read 16-byte vectors
        basis = tracker.shared(dtype=torch.float32)          # one tensor object per basis version: the views below are cached on it
        qb, qt = _basis_views(basis)
        coeff = stacr_ops.project(rows, qt)[:, : basis.shape[1]].to(torch.bfloat16)
        sparse = None
        if budget is not None and budget > 0:
            floor = 1.0 / rows.numel()                        # "at least one entry when the budget is positive"
            idx, packed = _select_residual_kernels(rows, coeff, qb, max(float(budget), floor), rows.shape[0], "global_topk", 16, 0.1, 0)
            if idx is not None:
                sparse = (idx, packed.data, packed.scale, packed.bits, packed.length)
        row_major = getattr(basis, "_sb_row_major", None)     # the rebuild kernel reads Q as contiguous fp32 [features, rank]
        if row_major is None:
            row_major = basis._sb_row_major = basis.contiguous()
        return PackedActivation(tuple(x.shape), x.dtype, coeff, row_major, sparse, codec=_KernelCodec.name)

    @staticmethod
    def decode(p: PackedActivation) -> torch.Tensor:
        from .ops import stacr_ops

        n_rows, width = p.coeff.shape[0], int(p.shape[-1])
        out = torch.empty(n_rows, width, dtype=torch.bfloat16, device=p.coeff.device)   # autograd keeps it: no shared scratch
        stacr_ops.rebuild_input(p.coeff, p.basis, p.residual, n_rows, width, out=out)
        return out.reshape(p.shape)


_CODECS = {c.name: c for c in (_FrameworkCodec, _KernelCodec)}


class STACRCompressor:
    """Pack/unpack hooks with one persistent Oja basis per (feature size, device)."""

    def __init__(self, config: STACRConfig | None = None):
        self.config = config or STACRConfig()
        self.step = 0
        self._trackers: dict[tuple[int, torch.device], OjaBasis] = {}

    # ---- step bookkeeping
    def set_step(self, step: int) -> None:
        self.step = int(step)

    def advance(self) -> None:
        self.step += 1

    # ---- which tensors are taken
    @staticmethod
    def is_parameter(t: torch.Tensor) -> bool:
        """Weights and biases, and views of them (autograd saves the transposed weight of a linear as a view)."""
        while t is not None:
            if isinstance(t, torch.nn.Parameter) or (t.requires_grad and t.is_leaf):
                return True
            t = getattr(t, "_base", None)
        return False

    def should_compress(self, t: torch.Tensor) -> bool:
        cfg = self.config
        if not t.is_floating_point() or t.dim() < 2 or self.is_parameter(t):
            return False
        return int(t.shape[-1]) >= int(cfg.min_features) and t.numel() >= int(cfg.min_numel)

    # ---- state
    def _tracker(self, t: torch.Tensor) -> OjaBasis:
        key = (int(t.shape[-1]), t.device)
        if key not in self._trackers:
            dtype = _resolve_basis_dtype(self.config.basis_dtype, t.dtype)
            self._trackers[key] = OjaBasis(key[0], self.config.rank, dtype=dtype, device=t.device)
        return self._trackers[key]

    def _budget_now(self) -> float | None:
        """The residual budget of this step, or ``None`` while the residual channel is off (mode ``none``, or turbo phase)."""
        cfg = self.config
        turbo = cfg.turbo_after_step is not None and self.step >= int(cfg.turbo_after_step)
        return None if (turbo or cfg.residual_mode == "none") else float(cfg.residual_budget)

    # ---- the hooks
    def pack(self, t: torch.Tensor) -> Any:
        cfg = self.config
        if self.step < int(cfg.warmup_steps) or not self.should_compress(t):
            return t
        x = t.detach()
        rows = x.reshape(-1, x.shape[-1])
        tracker = self._tracker(x)
        if self.step % max(1, int(cfg.update_interval)) == 0:
            tracker.update(rows, lr=float(cfg.oja_lr))
        codec = _KernelCodec if _KernelCodec.accepts(x, tracker.rank) else _FrameworkCodec
        return codec.encode(x, rows, tracker, self._budget_now())

    def unpack(self, packed: Any) -> torch.Tensor:
        if not isinstance(packed, PackedActivation):
            return packed
        return _CODECS[packed.codec].decode(packed)


@contextmanager
def stacr_saved_tensors(compressor: STACRCompressor):
    """Run a forward with the compressor installed as saved-tensor hooks."""
    with torch.autograd.graph.saved_tensors_hooks(compressor.pack, compressor.unpack):
        yield compressor
