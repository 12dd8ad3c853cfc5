"""Tensor-parallel GPT-2 by module replacement.

Column-parallel ``c_fc`` / ``c_attn`` (QKV cut per head, not contiguously), row-parallel ``c_proj``,
all-reduce placed between the row-parallel projection and dropout; embeddings, LayerNorms and the LM
head stay replicated.  Works on the in-tree ``GPT2LMHeadModel`` and on Hugging Face GPT-2 (Conv1D is
converted first).  API parity: stacr/protocols/tp_gpt2.py:34-501 of the reference project.  The
attention on the local heads runs through the fused flash kernel instead of materialising the
``S x S`` scores.
"""

from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

from ..parallel.tp import TPContext, column_parallel_linear, row_parallel_linear
from .tensor_parallel import (convert_conv1d_to_linear, copy_to_tp_region, reduce_from_tp_region, shard_linear_column,
                              shard_linear_row)


def shard_gpt2_qkv_column(linear: nn.Linear, tp_rank: int, tp_world_size: int, num_heads: int, head_dim: int) -> nn.Linear:
    """Shard fused ``[Q_all | K_all | V_all]`` rows so that each rank gets whole heads of Q, K and V."""
    if num_heads % tp_world_size:
        raise AssertionError(f"QKV shard: num_heads={num_heads} not divisible by tp_world_size={tp_world_size}")
    embed = num_heads * head_dim
    per = num_heads // tp_world_size * head_dim
    rows = torch.cat([torch.arange(part * embed + tp_rank * per, part * embed + (tp_rank + 1) * per) for part in range(3)])
    rows = rows.to(linear.weight.device)
    out = nn.Linear(linear.in_features, 3 * per, bias=linear.bias is not None, device=linear.weight.device, dtype=linear.weight.dtype)
    with torch.no_grad():
        out.weight.copy_(linear.weight[rows])
        if linear.bias is not None:
            out.bias.copy_(linear.bias[rows])
    return out


def _shard_call(layer, x, kind: str, group, fused: bool):
    """Run one tensor-parallel shard.  A plain ``nn.Linear`` goes through the functional fused forms; a compressed shard
    (the projection engine's ``STACRLinear``) is told its role once and then performs the collective inside its own GEMMs;
    any other wrapper keeps the explicit collectives around it."""
    from ..layers import STACRLinear

    if type(layer) is nn.Linear:
        fn = column_parallel_linear if kind == "column" else row_parallel_linear
        return fn(x, layer, group, fused)
    if isinstance(layer, STACRLinear):
        ctx = getattr(layer, "tp_context", None)
        if ctx is None or ctx.kind != kind or ctx.group is not group or ctx.fused != fused:
            layer.tp_context = TPContext(kind, group, fused)
        return layer(x)
    if kind == "column":
        return layer(copy_to_tp_region(x, group))
    return reduce_from_tp_region(layer(x), group)


def _find(module, *names, default=None):
    for n in names:
        if hasattr(module, n):
            return getattr(module, n)
    return default


class TPGPT2MLP(nn.Module):
    """copy -> c_fc (column) -> activation -> c_proj (row) -> all-reduce -> dropout."""

    def __init__(self, original_mlp, tp_rank, tp_world_size, tp_group):
        super().__init__()
        self.c_fc = shard_linear_column(original_mlp.c_fc, tp_rank, tp_world_size)
        self.c_proj = shard_linear_row(original_mlp.c_proj, tp_rank, tp_world_size)
        self.act = original_mlp.act
        self.dropout = _find(original_mlp, "dropout", default=nn.Identity())
        self.tp_group = tp_group
        self.fused_collectives = True

    def forward(self, hidden_states):
        x = _shard_call(self.c_fc, hidden_states, "column", self.tp_group, self.fused_collectives)
        x = self.act(x)
        return self.dropout(_shard_call(self.c_proj, x, "row", self.tp_group, self.fused_collectives))


class TPGPT2Attention(nn.Module):
    """Self-attention over this rank's heads; output projection is row-parallel."""

    def __init__(self, original_attn, tp_rank, tp_world_size, tp_group):
        super().__init__()
        heads = int(_find(original_attn, "n_head", "num_heads"))
        head_dim = int(_find(original_attn, "head_dim"))
        self.local_heads, self.head_dim = heads // tp_world_size, head_dim
        self.c_attn = shard_gpt2_qkv_column(original_attn.c_attn, tp_rank, tp_world_size, heads, head_dim)
        self.c_proj = shard_linear_row(original_attn.c_proj, tp_rank, tp_world_size)
        drop = _find(original_attn, "attn_dropout")
        self.attn_pdrop = float(_find(original_attn, "attn_pdrop", default=getattr(drop, "p", 0.0)))
        self.resid_dropout = _find(original_attn, "resid_dropout", default=nn.Identity())
        self.tp_group = tp_group
        self.fused_collectives = True

    def forward(self, hidden_states, attention_mask=None, **kwargs):
        b, s, _ = hidden_states.shape
        qkv = _shard_call(self.c_attn, hidden_states, "column", self.tp_group, self.fused_collectives)
        x = hidden_states
        q, k, v = qkv.split(self.local_heads * self.head_dim, dim=-1)
        shape = lambda t: t.view(b, s, self.local_heads, self.head_dim).transpose(1, 2)
        mask = None
        if attention_mask is not None and attention_mask.dim() == 2 and not bool(attention_mask.all()):
            mask = attention_mask[:, None, None, :].bool() & torch.ones(s, s, dtype=torch.bool, device=x.device).tril()
        ctx = F.scaled_dot_product_attention(shape(q), shape(k), shape(v), attn_mask=mask, is_causal=mask is None,
                                             dropout_p=self.attn_pdrop if self.training else 0.0)
        merged = ctx.transpose(1, 2).reshape(b, s, self.local_heads * self.head_dim)
        out = self.resid_dropout(_shard_call(self.c_proj, merged, "row", self.tp_group, self.fused_collectives))
        if kwargs.get("output_attentions") is not None or kwargs.get("use_cache") is not None or "layer_past" in kwargs:
            return out, None  # Hugging Face block expects a tuple
        return out


def apply_tensor_parallel_gpt2(model, tp_rank, tp_world_size, tp_group=None, scope="mlp_only", verbose=False):
    """Replace the MLP (and, with ``scope='full'``, the attention) of every block by its sharded form."""
    if scope not in ("mlp_only", "full"):
        raise ValueError(f"Unknown TP scope: {scope!r}. Use 'mlp_only' or 'full'.")
    heads = model.config.n_head
    if scope == "full" and heads % tp_world_size:
        valid = [d for d in range(1, heads + 1) if heads % d == 0]
        raise ValueError(f"num_heads={heads} is not divisible by tp_world_size={tp_world_size}. GPT-2 TP requires "
                         f"num_heads % tp_world_size == 0. For this model, valid TP degrees are: {valid}")
    converted = convert_conv1d_to_linear(model)
    for block in model.transformer.h:
        block.mlp = TPGPT2MLP(block.mlp, tp_rank, tp_world_size, tp_group)
        if scope == "full":
            block.attn = TPGPT2Attention(block.attn, tp_rank, tp_world_size, tp_group)
    drop = getattr(model.transformer, "drop", None)
    if isinstance(drop, nn.Dropout):
        drop.p = 0.0  # no synchronised dropout on the replicated path
    if verbose and tp_rank == 0:
        n = sum(p.numel() for p in model.parameters())
        print(f"[TP] converted {converted} Conv1D, sharded {len(model.transformer.h)} blocks (scope={scope}); {n:,} parameters per rank")
    return model


def get_tp_stacr_targets(model, tp_stacr_scope="row_only"):
    """Names of the sharded linears to compress: ``row_only`` | ``all_mlp`` | ``all_linear``."""
    patterns = {"row_only": ("mlp.c_proj",), "all_mlp": ("mlp.c_fc", "mlp.c_proj"),
                "all_linear": ("mlp.c_fc", "mlp.c_proj", "attn.c_attn", "attn.c_proj")}
    if tp_stacr_scope not in patterns:
        raise ValueError(f"Unknown tp_stacr_scope: {tp_stacr_scope}. Must be one of {tuple(patterns)}")
    want = patterns[tp_stacr_scope]
    return [n for n, m in model.named_modules() if isinstance(m, nn.Linear) and any(p in n for p in want)]


def disable_tp_dropout(model) -> int:
    """Zero every dropout probability (ranks would otherwise draw different masks)."""
    count = 0
    for m in model.modules():
        if isinstance(m, nn.Dropout) and m.p > 0:
            m.p = 0.0
            count += 1
    return count


class TPActivationProfiler:
    """Forward-hook census of activation bytes entering each projection family (replicated vs sharded inputs)."""

    FAMILIES = ("mlp.c_fc", "mlp.c_proj", "attn.c_attn", "attn.c_proj")

    def __init__(self, model):
        self.bytes = {f: 0 for f in self.FAMILIES}
        self.calls = {f: 0 for f in self.FAMILIES}
        self._handles = []
        for name, module in model.named_modules():
            for fam in self.FAMILIES:
                if name.endswith(fam):
                    self._handles.append(module.register_forward_hook(self._hook(fam)))

    def _hook(self, fam):
        def fn(_module, inputs, _output):
            x = inputs[0]
            self.bytes[fam] += x.numel() * x.element_size()
            self.calls[fam] += 1
        return fn

    def summary(self) -> dict:
        total = sum(self.bytes.values())
        return {"bytes": dict(self.bytes), "calls": dict(self.calls), "total_bytes": total,
                "share": {f: (b / total if total else 0.0) for f, b in self.bytes.items()}}

    def close(self):
        for h in self._handles:
            h.remove()
        self._handles = []
