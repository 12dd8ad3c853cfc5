"""Low-rank adapters (LoRA) and a 4-bit NormalFloat frozen base (QLoRA) for the adapter-composition grids.

The composition question these grids ask: when only adapters train, which saved activations are left for STAC-R to
compress?  With adapters on the attention projections and a frozen MLP, none of the MLP inputs is saved for a weight
gradient, so the compression surface is *empty* (the negative-composition control); with full training it is the
whole MLP.  The reference answers with ``peft`` and ``bitsandbytes`` (experiments/benchmarks/lora.py:38-124,
qlora.py:35-110); neither is needed here.

``LoRALinear``  ``y = base(x) + (alpha / r) * (x Aᵀ) Bᵀ`` with ``A`` Kaiming-uniform, ``B`` zero, base frozen.
``NF4Linear``   frozen weight stored as 4-bit NormalFloat codes with one absmax per 64 values, the absmaxes themselves
                quantised to 8 bits per 256 (double quantisation); dequantised on the fly in forward and again in
                backward, so that no full-precision copy of the weight is kept between the two.
"""

from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch
from torch import nn
from torch.nn import functional as F

# The 16 NormalFloat-4 levels: quantiles of N(0, 1) normalised to [-1, 1], with an exact zero (QLoRA, Dettmers et al., 2023).
NF4_LEVELS = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635, -0.18477343022823334,
              -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
              0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0)
BLOCK, SCALE_BLOCK = 64, 256


def nf4_quantize(weight: torch.Tensor):
    """``(codes uint8 [n/2], scale_codes uint8, scale_scale fp32, scale_mean fp32)`` of a flattened weight (padded to 64)."""
    flat = weight.detach().float().reshape(-1)
    pad = (-flat.numel()) % BLOCK
    flat = F.pad(flat, (0, pad)).view(-1, BLOCK)
    absmax = flat.abs().amax(dim=1).clamp_min(1e-12)
    levels = torch.tensor(NF4_LEVELS, device=flat.device)
    codes = ((flat / absmax[:, None])[..., None] - levels).abs().argmin(dim=-1).to(torch.uint8).view(-1)
    packed = (codes[0::2] << 4) | codes[1::2]
    mean = absmax.mean()
    centred = absmax - mean
    spad = (-centred.numel()) % SCALE_BLOCK
    blocks = F.pad(centred, (0, spad)).view(-1, SCALE_BLOCK)
    sscale = blocks.abs().amax(dim=1).clamp_min(1e-12) / 127.0
    scodes = torch.round(blocks / sscale[:, None]).clamp(-127, 127).to(torch.int8).view(-1)[:centred.numel()]
    return packed, scodes, sscale, mean


def nf4_dequantize(packed, scodes, sscale, mean, shape, dtype=torch.float32) -> torch.Tensor:
    n = math.prod(shape)
    levels = torch.tensor(NF4_LEVELS, device=packed.device, dtype=torch.float32)
    codes = torch.stack([(packed >> 4) & 0xF, packed & 0xF], dim=1).view(-1).long()
    spad = (-scodes.numel()) % SCALE_BLOCK
    absmax = (F.pad(scodes.float(), (0, spad)).view(-1, SCALE_BLOCK) * sscale[:, None]).view(-1)[:scodes.numel()] + mean
    values = levels[codes].view(-1, BLOCK) * absmax[:, None]
    return values.view(-1)[:n].view(shape).to(dtype)


class _NF4Matmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        ctx.layer = layer
        return F.linear(x, layer.dequantize(x.dtype))

    @staticmethod
    def backward(ctx, dy):
        return dy @ ctx.layer.dequantize(dy.dtype), None


class NF4Linear(nn.Module):
    """Frozen linear layer whose weight lives as NF4 codes (about 4.13 bits per weight with double quantisation)."""

    def __init__(self, source: nn.Linear):
        super().__init__()
        self.in_features, self.out_features = source.in_features, source.out_features
        packed, scodes, sscale, mean = nf4_quantize(source.weight)
        self.register_buffer("codes", packed)
        self.register_buffer("scale_codes", scodes)
        self.register_buffer("scale_scale", sscale)
        self.register_buffer("scale_mean", mean)
        self.bias = None if source.bias is None else nn.Parameter(source.bias.detach().clone(), requires_grad=False)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return nf4_dequantize(self.codes, self.scale_codes, self.scale_scale, self.scale_mean, (self.out_features, self.in_features), dtype)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.codes, self.scale_codes, self.scale_scale, self.scale_mean))

    def forward(self, x):
        y = _NF4Matmul.apply(x, self) if x.requires_grad else F.linear(x, self.dequantize(x.dtype))
        return y if self.bias is None else y + self.bias.to(y.dtype)


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Module, r: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        self.base, self.r, self.scaling = base, int(r), float(alpha) / int(r)
        self.in_features, self.out_features = base.in_features, base.out_features
        for p in base.parameters():
            p.requires_grad_(False)
        ref = next(base.parameters(), None)
        kw = {"device": ref.device if ref is not None else None, "dtype": ref.dtype if ref is not None and ref.is_floating_point() else None}
        if isinstance(base, NF4Linear):
            kw = {"device": base.codes.device, "dtype": torch.float32}
        self.lora_A = nn.Parameter(torch.empty(self.r, self.in_features, **kw))
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, self.r, **kw))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x):
        update = F.linear(F.linear(self.dropout(x), self.lora_A.to(x.dtype)), self.lora_B.to(x.dtype))
        return self.base(x) + self.scaling * update

    def merged_weight(self) -> torch.Tensor:
        base = self.base.dequantize() if isinstance(self.base, NF4Linear) else self.base.weight
        return base + self.scaling * (self.lora_B @ self.lora_A).to(base.dtype)


def default_targets(model: nn.Module) -> List[str]:
    """Attention projections the adapter grids use: ``query``/``value`` for BERT-style encoders, fused ``c_attn`` for GPT-2,
    ``q_proj``/``v_proj`` for LLaMA-style and ``query_key_value`` for NeoX-style decoders."""
    leaves = {name.rsplit(".", 1)[-1] for name, m in model.named_modules() if isinstance(m, nn.Linear)}
    for group in (("query", "value"), ("c_attn",), ("q_proj", "v_proj"), ("query_key_value",)):
        if all(g in leaves for g in group):
            return list(group)
    raise ValueError("no known attention projection names in this model; pass target_modules")


def apply_lora(model: nn.Module, target_modules: Optional[Iterable[str]] = None, r: int = 8, alpha: float = 16.0, dropout: float = 0.0,
               quantize_base: bool = False, train_head: bool = False) -> List[LoRALinear]:
    """Freeze the model, put adapters on linears whose leaf name is in ``target_modules``; with ``quantize_base`` every other
    linear inside the transformer blocks (and the adapted ones' bases) becomes an :class:`NF4Linear`.  Returns the adapters."""
    from ..composition import transformer_blocks

    targets = set(target_modules or default_targets(model))
    for p in model.parameters():
        p.requires_grad_(False)
    in_blocks = {id(m) for blk in transformer_blocks(model) for m in blk.modules()}
    adapters = []
    for name, module in list(model.named_modules()):
        if not isinstance(module, nn.Linear) or id(module) not in in_blocks:
            continue
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        base = NF4Linear(module) if quantize_base else module
        if leaf in targets:
            adapter = LoRALinear(base, r, alpha, dropout)
            setattr(parent, leaf, adapter)
            adapters.append(adapter)
        elif quantize_base:
            setattr(parent, leaf, base)
    if not adapters:
        raise ValueError(f"no linear layer matched target_modules={sorted(targets)}")
    if train_head:
        for name, p in model.named_parameters():
            if any(h in name for h in ("classifier", "score", "lm_head")):
                p.requires_grad_(True)
    return adapters


def trainable_parameter_report(model: nn.Module) -> dict:
    total = sum(p.numel() for p in model.parameters())
    train = sum(p.numel() for p in model.parameters() if p.requires_grad)
    quant = sum(m.weight_bytes() for m in model.modules() if isinstance(m, NF4Linear))
    return {"parameters": total, "trainable_parameters": train, "trainable_pct": 100.0 * train / max(total, 1), "nf4_weight_bytes": quant}
