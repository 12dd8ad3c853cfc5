"""GPT-NeoX / Pythia decoder: rotary embedding on a fraction of each head, parallel attention+MLP residual."""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

import os

from ..ops import attention as attention_ops
from ..ops import nn_ops
from .common import _attention_engine as attention_engine, causal_attention, Embedding, GELU, init_weights, LayerNorm, Linear, lm_loss, ModelOutput


_FUSED_NORMS = os.environ.get("STACR_FUSED_NORMS", "1") == "1"   # 0: the two norms and the residual sum as separate ops


@dataclass
class NeoXConfig:
    vocab_size: int = 50304
    hidden_size: int = 2048
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 8192
    rotary_pct: float = 0.25
    rotary_emb_base: float = 10000.0
    max_position_embeddings: int = 2048
    layer_norm_eps: float = 1e-5
    use_parallel_residual: bool = True
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    tie_word_embeddings: bool = False
    loss_chunk: int = 0


PRESETS = {
    "pythia-70m": dict(hidden_size=512, num_hidden_layers=6, num_attention_heads=8, intermediate_size=2048),
    "pythia-160m": dict(hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072),
    "pythia-410m": dict(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096),
    "pythia-1b": dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=8, intermediate_size=8192),
    "pythia-1.4b": dict(hidden_size=2048, num_hidden_layers=24, num_attention_heads=16, intermediate_size=8192),
    "pythia-2.8b": dict(hidden_size=2560, num_hidden_layers=32, num_attention_heads=32, intermediate_size=10240),
}


def rotary_tables(seq: int, dim: int, base: float, device, dtype=torch.float32):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rotary(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot: int) -> torch.Tensor:
    """Rotate the first ``rot`` dims of each head (``[B, H, S, D]``); the rest pass through."""
    tr, tp = t[..., :rot], t[..., rot:]
    half = rot // 2
    rotated = torch.cat((-tr[..., half:], tr[..., :half]), dim=-1)
    return torch.cat((tr * cos + rotated * sin, tp), dim=-1)


class NeoXAttention(nn.Module):
    def __init__(self, cfg: NeoXConfig):
        super().__init__()
        self.n_head = cfg.num_attention_heads
        self.head_dim = cfg.hidden_size // cfg.num_attention_heads
        self.rot = int(self.head_dim * cfg.rotary_pct)
        self.base = cfg.rotary_emb_base
        self.query_key_value = Linear(cfg.hidden_size, 3 * cfg.hidden_size)
        self.dense = Linear(cfg.hidden_size, cfg.hidden_size)
        self.attention_dropout = cfg.attention_dropout
        self._tables = None
        self._half = None

    def _rotary(self, seq, device, dtype):
        key = (seq, device, dtype)
        if self._tables is None or self._tables[0] != key:
            self._tables = (key, rotary_tables(seq, self.rot, self.base, device, dtype))
        return self._tables[1]

    def _half_tables(self, seq, device):
        key = ("half", seq, device)
        if self._half is None or self._half[0] != key:
            inv = 1.0 / (self.base ** (torch.arange(0, self.rot, 2, device=device, dtype=torch.float32) / self.rot))
            ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
            self._half = (key, ang.cos().contiguous(), ang.sin().contiguous())
        return self._half[1], self._half[2]

    def forward(self, x, attention_mask=None):
        b, s, d = x.shape
        # project the flattened tokens: the 2-D result is a tensor of its own, whereas the 3-D form would be a VIEW of it,
        # and an in-place op on a view makes autograd re-materialise the base (three extra copies of qkv per layer)
        qkv = self.query_key_value(x.reshape(b * s, d))
        if nn_ops.rotary_qk_supported(qkv, self.head_dim, self.rot):
            cos, sin = self._half_tables(s, x.device)
            qkv = nn_ops.rotary_qk(qkv, cos, sin, s, self.n_head, self.head_dim, self.rot)  # fused, in place
            if (attention_engine() == "intree" and attention_ops.fused_supported(qkv, self.head_dim)
                    and not (self.training and self.attention_dropout > 0.0)):
                # in-tree forward and backward straight on the fused projection: no split, cat or transpose copies
                mask = attention_mask if attention_mask is not None and not bool(attention_mask.all()) else None
                ctx = attention_ops.fused_qkv_attention(qkv, b, s, self.n_head, self.head_dim, layout="interleaved", causal=True, key_mask=mask)
                return self.dense(ctx)
            q, k, v = (t.transpose(1, 2) for t in qkv.view(b, s, self.n_head, 3 * self.head_dim).split(self.head_dim, dim=-1))
        else:
            # NeoX interleaves per head: [H, 3 * head_dim]
            q, k, v = (t.transpose(1, 2) for t in qkv.view(b, s, self.n_head, 3 * self.head_dim).split(self.head_dim, dim=-1))
            cos, sin = self._rotary(s, x.device, q.dtype)
            q, k = apply_rotary(q, cos, sin, self.rot), apply_rotary(k, cos, sin, self.rot)
        ctx = causal_attention(q, k, v, causal=True, attention_mask=attention_mask, dropout_p=self.attention_dropout, training=self.training)
        return self.dense(ctx.transpose(1, 2).reshape(b, s, d))


class NeoXMLP(nn.Module):
    def __init__(self, cfg: NeoXConfig):
        super().__init__()
        self.dense_h_to_4h = Linear(cfg.hidden_size, cfg.intermediate_size)
        self.act = GELU("none")
        self.dense_4h_to_h = Linear(cfg.intermediate_size, cfg.hidden_size)

    def forward(self, x):
        return self.dense_4h_to_h(self.act(self.dense_h_to_4h(x)))


class NeoXLayer(nn.Module):
    def __init__(self, cfg: NeoXConfig):
        super().__init__()
        self.parallel = cfg.use_parallel_residual
        self.input_layernorm = LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.post_attention_layernorm = LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.attention = NeoXAttention(cfg)
        self.mlp = NeoXMLP(cfg)
        self.drop = nn.Dropout(cfg.hidden_dropout)

    def forward(self, x, attention_mask=None):
        ln1, ln2 = self.input_layernorm, self.post_attention_layernorm
        hooked = ln1._forward_hooks or ln1._forward_pre_hooks or ln2._forward_hooks or ln2._forward_pre_hooks
        if (self.parallel and not hooked and _FUSED_NORMS and ln1.eps == ln2.eps and type(ln1) is LayerNorm and type(ln2) is LayerNorm
                and nn_ops.parallel_norms_supported(x, ln1.weight, ln1.bias, ln2.weight, ln2.bias)):
            # both branches normalise the same x: one kernel forward, and one kernel backward for the three gradients
            # (two branches + residual) that meet at x
            h1, h2, skip = nn_ops.parallel_layer_norms(x, ln1.weight, ln1.bias, ln2.weight, ln2.bias, ln1.eps)
            return nn_ops.add3(skip, self.drop(self.attention(h1, attention_mask)), self.drop(self.mlp(h2)))
        attn = self.drop(self.attention(self.input_layernorm(x), attention_mask))
        if self.parallel:  # x + attn(ln1(x)) + mlp(ln2(x))
            return x + attn + self.drop(self.mlp(self.post_attention_layernorm(x)))
        x = x + attn
        return x + self.drop(self.mlp(self.post_attention_layernorm(x)))


class NeoXModel(nn.Module):
    def __init__(self, cfg: NeoXConfig):
        super().__init__()
        self.embed_in = Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(NeoXLayer(cfg) for _ in range(cfg.num_hidden_layers))
        self.final_layer_norm = LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)

    def forward(self, input_ids, attention_mask=None):
        x = self.embed_in(input_ids)
        if torch.is_autocast_enabled(x.device.type):
            x = x.to(torch.get_autocast_dtype(x.device.type))
        for layer in self.layers:
            x = layer(x, attention_mask)
        return self.final_layer_norm(x)


class GPTNeoXForCausalLM(nn.Module):
    def __init__(self, cfg: NeoXConfig):
        super().__init__()
        self.config = cfg
        self.gpt_neox = NeoXModel(cfg)
        self.embed_out = Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.apply(init_weights)
        if cfg.tie_word_embeddings:
            self.embed_out.weight = self.gpt_neox.embed_in.weight

    def forward(self, input_ids, attention_mask=None, labels=None, **_):
        hidden = self.gpt_neox(input_ids, attention_mask)
        if labels is not None and self.config.loss_chunk:
            return ModelOutput(loss=lm_loss(hidden, labels, self.embed_out, self.config.loss_chunk))
        logits = self.embed_out(hidden)
        loss = lm_loss(logits, labels) if labels is not None else None
        return ModelOutput(loss=loss, logits=logits)
