"""Compression of the attention surface (Q/K/V/output projections) with the adaptive engine.

* mask-aware wrapping: padded tokens are dropped before compression and scattered back afterwards, so they
  neither pollute the tracked subspace nor consume residual budget;
* joint Q/K: the query and key projections read the same input, so they can share one basis (one pooled
  basis object, half the basis memory and one update per step);
* GPT-2's fused ``c_attn`` can be split into three compressed projections over the same input.

Parity: stacr/protocols/attention.py:18-733 of the reference project.
"""

from __future__ import annotations

import threading
from contextlib import contextmanager
from dataclasses import dataclass, field
from functools import wraps
from typing import List, Optional

import torch
from torch import nn

from ..adaptive import STACRConfig, STACRLinear, _TransposedProjection, get_basis_pool

_MASK = threading.local()


def _get_current_attention_mask() -> Optional[torch.Tensor]:
    return getattr(_MASK, "mask", None)


@contextmanager
def _attention_mask_context(mask: Optional[torch.Tensor]):
    outer = getattr(_MASK, "mask", None)
    _MASK.mask = mask
    try:
        yield
    finally:
        _MASK.mask = outer


def _extract_token_mask(attention_mask: Optional[torch.Tensor], seq_len: int, device) -> Optional[torch.Tensor]:
    """Boolean ``[B, S]`` mask of real tokens from a 2-D binary mask or a 3/4-D (additive or boolean) mask."""
    if attention_mask is None:
        return None
    m = attention_mask
    if m.dim() not in (2, 3, 4) or m.size(-1) != seq_len:
        return None
    if m.dtype.is_floating_point:
        keep = (m >= 0) if (m.dim() > 2 or bool((m < 0).any())) else (m != 0)
    else:
        keep = m != 0
    if m.dim() > 2:
        # a key position is real if any query may attend to it (row 0 of a causal mask would hide later tokens)
        keep = keep.reshape(m.shape[0], -1, seq_len).any(dim=1)
    return keep.to(device)


def _wrap_attention_forward(module: nn.Module) -> None:
    """Publish the attention mask of each call of ``module.forward`` to the wrapped projections underneath."""
    if getattr(module, "_stacr_mask_wrapped", False):
        return
    inner = module.forward

    @wraps(inner)
    def forward(*args, **kwargs):
        mask = kwargs.get("attention_mask")
        if mask is None:
            mask = next((a for a in args[1:] if isinstance(a, torch.Tensor) and a.dim() in (2, 3, 4) and a.dtype != torch.long), None)
        with _attention_mask_context(mask):
            return inner(*args, **kwargs)

    module.forward = forward
    module._stacr_mask_wrapped = True


class _GatherRows(torch.autograd.Function):
    """``flat[rows]`` and its adjoint (scatter into zeros) on the row-move kernel for bf16 CUDA matrices."""

    @staticmethod
    def forward(ctx, flat, rows):
        from ..ops import pack_ops

        ctx.save_for_backward(rows)
        ctx.total = flat.shape[0]
        return pack_ops.move_rows(flat.contiguous(), rows)

    @staticmethod
    def backward(ctx, grad):
        from ..ops import pack_ops

        (rows,) = ctx.saved_tensors
        full = torch.zeros(ctx.total, grad.shape[1], dtype=grad.dtype, device=grad.device)
        return pack_ops.move_rows(grad.contiguous(), rows, scatter_into=full), None


class _ScatterRows(torch.autograd.Function):
    """Rows placed into a zero matrix of ``total`` rows, and the adjoint (gather), on the same kernel."""

    @staticmethod
    def forward(ctx, src, rows, total):
        from ..ops import pack_ops

        ctx.save_for_backward(rows)
        full = torch.zeros(total, src.shape[1], dtype=src.dtype, device=src.device)
        return pack_ops.move_rows(src.contiguous(), rows, scatter_into=full)

    @staticmethod
    def backward(ctx, grad):
        from ..ops import pack_ops

        (rows,) = ctx.saved_tensors
        return pack_ops.move_rows(grad.contiguous(), rows), None, None


def _rows_on_kernels(t: torch.Tensor) -> bool:
    from ..ops import _lib

    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] % 8 == 0 and _lib.available()


def gather_rows(flat: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    return _GatherRows.apply(flat, rows) if _rows_on_kernels(flat) else flat.index_select(0, rows)


def scatter_rows(src: torch.Tensor, rows: torch.Tensor, total: int) -> torch.Tensor:
    if _rows_on_kernels(src):
        return _ScatterRows.apply(src, rows, total)
    return torch.zeros(total, src.shape[1], dtype=src.dtype, device=src.device).index_copy(0, rows, src)


class _MaskAwareSTACRLinear(nn.Module):
    """Runs the wrapped compressed layer on real tokens only."""

    def __init__(self, inner: STACRLinear):
        super().__init__()
        self.inner = inner

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        mask = _get_current_attention_mask()
        keep = _extract_token_mask(mask, x.shape[1], x.device) if (mask is not None and x.dim() == 3) else None
        if keep is None or bool(keep.all()):
            return self.inner(x)
        flat = x.reshape(-1, x.shape[-1])
        rows = keep.reshape(-1).nonzero(as_tuple=False).reshape(-1)
        if rows.numel() == 0:
            return x.new_zeros(x.shape[0], x.shape[1], self.inner.out_features)
        out_rows = self.inner(gather_rows(flat, rows))
        out = scatter_rows(out_rows, rows, flat.shape[0])
        return out.view(x.shape[0], x.shape[1], -1)

    def __getattr__(self, name: str):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.inner, name)


_JOINT_GROUP_BASE = 1_000_000


class JointQKSTACRLinear(nn.Module):
    """Query and key projections compressed against one shared basis (a pooled basis object)."""

    def __init__(self, query: nn.Module, key: nn.Module, config: STACRConfig, *, mask_aware: bool = False, layer_index: int = 0):
        super().__init__()
        if config.rank_mode != "fixed":
            raise ValueError("joint Q/K requires rank_mode='fixed'")
        opts = {**config.to_dict(), "basis_sharing": "all", "basis_sharing_group": _JOINT_GROUP_BASE + int(layer_index), "joint_qk": False}
        q = STACRLinear.from_linear(query, STACRConfig(**opts), layer_index=layer_index)
        k = STACRLinear.from_linear(key, STACRConfig(**opts), layer_index=layer_index)
        self.query = _MaskAwareSTACRLinear(q) if mask_aware else q
        self.key = _MaskAwareSTACRLinear(k) if mask_aware else k

    def shared_basis(self) -> torch.Tensor:
        q = self.query.inner if isinstance(self.query, _MaskAwareSTACRLinear) else self.query
        return q._resolve_basis()

    def forward(self, x: torch.Tensor):
        return self.query(x), self.key(x)


class _SliceLinear(nn.Module):
    """A view of rows ``[lo, hi)`` of a fused projection as a standalone linear (parameters are views, not copies)."""

    def __init__(self, source: nn.Module, lo: int, hi: int, conv1d: bool):
        super().__init__()
        self.source, self.lo, self.hi, self.conv1d = source, lo, hi, conv1d
        self.in_features = int(source.weight.shape[0] if conv1d else source.weight.shape[1])
        self.out_features = hi - lo

    @property
    def weight(self):
        w = self.source.weight
        return w[:, self.lo:self.hi].t() if self.conv1d else w[self.lo:self.hi]

    @property
    def bias(self):
        b = getattr(self.source, "bias", None)
        return None if b is None else b[self.lo:self.hi]

    def forward(self, x):
        return torch.nn.functional.linear(x, self.weight, self.bias)


class _SplitQKVWrapper(nn.Module):
    """Replaces GPT-2's fused ``c_attn``: three compressed projections whose outputs are concatenated."""

    def __init__(self, c_attn: nn.Module, config: STACRConfig, *, mask_aware: bool = False, layer_index: int = 0):
        super().__init__()
        conv1d = type(c_attn).__name__ == "Conv1D"
        total = int(c_attn.weight.shape[1] if conv1d else c_attn.weight.shape[0])
        if total % 3:
            raise ValueError("fused QKV width must be divisible by 3")
        part = total // 3
        self.source = c_attn
        layers = []
        for i in range(3):
            sl = _SliceLinear(c_attn, i * part, (i + 1) * part, conv1d)
            layer = _SlicedSTACR(sl, STACRConfig(**config.to_dict()), layer_index=layer_index * 3 + i)
            layers.append(_MaskAwareSTACRLinear(layer) if mask_aware else layer)
        self.q_layer, self.k_layer, self.v_layer = layers

    def forward(self, x):
        return torch.cat((self.q_layer(x), self.k_layer(x), self.v_layer(x)), dim=-1)


class _SlicedSTACR(STACRLinear):
    """Adaptive layer over a weight slice: the slice is re-read every forward so the fused parameter keeps training."""

    def __init__(self, sliced: _SliceLinear, config: STACRConfig, layer_index: int = 0):
        super().__init__(sliced.in_features, sliced.out_features, config, layer_index=layer_index, _linear=sliced)
        self.train(sliced.source.training)


@dataclass
class AttentionCompressionReport:
    replaced: int = 0
    skipped: int = 0
    joint_qk_pairs: int = 0
    warnings: List[str] = field(default_factory=list)
    layer_names: List[str] = field(default_factory=list)

    def to_dict(self) -> dict:
        return {"replaced": self.replaced, "skipped": self.skipped, "joint_qk_pairs": self.joint_qk_pairs, "warnings": list(self.warnings),
                "layer_names": list(self.layer_names)}


_TRIPLES = (("query", "key", "value"), ("q_proj", "k_proj", "v_proj"))
_COMPRESSED = (STACRLinear, _MaskAwareSTACRLinear, JointQKSTACRLinear, _SplitQKVWrapper)


def _linear_like(m) -> bool:
    return isinstance(m, nn.Linear) or type(m).__name__ == "Conv1D"


def apply_stacr_to_attention(model: nn.Module, config: STACRConfig, *, enable_gpt2_c_attn_split: bool = False, mask_aware: bool = False,
                             joint_qk: bool = False) -> AttentionCompressionReport:
    """Wrap Q/K/V projections (``query/key/value``, ``q_proj/k_proj/v_proj`` or, opt-in, GPT-2's ``c_attn``)."""
    report = AttentionCompressionReport()
    if joint_qk and config.rank_mode != "fixed":
        report.warnings.append(f"joint_qk only supports rank_mode='fixed'; disabling joint_qk for rank_mode={config.rank_mode!r}.")
        joint_qk = False
    index = 0
    for name, module in list(model.named_modules()):
        if isinstance(module, _COMPRESSED):
            continue
        triple = next((t for t in _TRIPLES if all(hasattr(module, a) for a in t)), None)
        if triple is not None:
            q_name, k_name, v_name = triple
            q, k, v = (getattr(module, a) for a in triple)
            if any(isinstance(p, _COMPRESSED) for p in (q, k, v)) or not all(_linear_like(p) for p in (q, k, v)):
                report.skipped += 1
                continue
            if mask_aware:
                _wrap_attention_forward(module)
            if joint_qk:
                joint = JointQKSTACRLinear(q, k, config, mask_aware=mask_aware, layer_index=index)
                setattr(module, q_name, joint.query)
                setattr(module, k_name, joint.key)
                module._joint_qk_wrapper = joint
                report.joint_qk_pairs += 1
                report.replaced += 2
                index += 1
                rest = (v_name,)
            else:
                rest = triple
            for attr in rest:
                layer = STACRLinear.from_linear(getattr(module, attr), STACRConfig(**config.to_dict()), layer_index=index)
                layer.source_name = f"{name}.{attr}"
                setattr(module, attr, _MaskAwareSTACRLinear(layer) if mask_aware else layer)
                report.layer_names.append(layer.source_name)
                report.replaced += 1
                index += 1
        elif hasattr(module, "c_attn") and _linear_like(module.c_attn):
            if not enable_gpt2_c_attn_split:
                report.skipped += 1
                report.warnings.append(f"{name}.c_attn is fused; pass enable_gpt2_c_attn_split=True to compress it")
                continue
            if mask_aware:
                _wrap_attention_forward(module)
            module.c_attn = _SplitQKVWrapper(module.c_attn, config, mask_aware=mask_aware, layer_index=index)
            report.layer_names.append(f"{name}.c_attn")
            report.replaced += 3
            index += 1
    if joint_qk and not report.joint_qk_pairs:
        report.warnings.append("joint_qk requested but no separate query/key projections were found")
    return report


def clear_joint_qk_bases() -> None:
    get_basis_pool().clear()
