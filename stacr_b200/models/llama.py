"""LLaMA / Qwen-style decoder: RMSNorm, full rotary embedding, grouped-query attention, SwiGLU MLP."""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn
from torch.nn import functional as F

from .common import causal_attention, Embedding, init_weights, Linear, lm_loss, ModelOutput
from .neox import apply_rotary, rotary_tables


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 2048
    num_hidden_layers: int = 16
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    intermediate_size: int = 8192
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    loss_chunk: int = 0


PRESETS = {
    "llama-tiny": dict(vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=688, max_position_embeddings=256),
    "llama-3.2-1b": dict(vocab_size=128256, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, intermediate_size=8192, rope_theta=500000.0, tie_word_embeddings=True),
    "llama-3.2-3b": dict(vocab_size=128256, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, num_key_value_heads=8, intermediate_size=8192, rope_theta=500000.0, tie_word_embeddings=True),
    "llama-3.1-8b": dict(vocab_size=128256, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, intermediate_size=14336, rope_theta=500000.0),
    "qwen2.5-1.5b": dict(vocab_size=151936, hidden_size=1536, num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960, rope_theta=1000000.0, attention_bias=True, tie_word_embeddings=True),
    "qwen2.5-7b": dict(vocab_size=152064, hidden_size=3584, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, rope_theta=1000000.0, attention_bias=True),
    "qwen2.5-14b": dict(vocab_size=152064, hidden_size=5120, num_hidden_layers=48, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824, rope_theta=1000000.0, attention_bias=True),
}


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        var = x.float().square().mean(-1, keepdim=True)
        return (x.float() * torch.rsqrt(var + self.eps)).to(x.dtype) * self.weight.to(x.dtype)


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.n_head, self.n_kv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.head_dim = cfg.hidden_size // cfg.num_attention_heads
        self.theta = cfg.rope_theta
        self.q_proj = Linear(cfg.hidden_size, self.n_head * self.head_dim, bias=cfg.attention_bias)
        self.k_proj = Linear(cfg.hidden_size, self.n_kv * self.head_dim, bias=cfg.attention_bias)
        self.v_proj = Linear(cfg.hidden_size, self.n_kv * self.head_dim, bias=cfg.attention_bias)
        self.o_proj = Linear(self.n_head * self.head_dim, cfg.hidden_size, bias=False)
        self._tables = None

    def forward(self, x, attention_mask=None):
        b, s, _ = x.shape
        q = self.q_proj(x).view(b, s, self.n_head, self.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(b, s, self.n_kv, self.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(b, s, self.n_kv, self.head_dim).transpose(1, 2)
        key = (s, x.device, q.dtype)
        if self._tables is None or self._tables[0] != key:
            self._tables = (key, rotary_tables(s, self.head_dim, self.theta, x.device, q.dtype))
        cos, sin = self._tables[1]
        q, k = apply_rotary(q, cos, sin, self.head_dim), apply_rotary(k, cos, sin, self.head_dim)
        if self.n_kv != self.n_head:
            rep = self.n_head // self.n_kv
            k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        ctx = causal_attention(q, k, v, causal=True, attention_mask=attention_mask)
        return self.o_proj(ctx.transpose(1, 2).reshape(b, s, -1))


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.gate_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.self_attn = LlamaAttention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mlp = LlamaMLP(cfg)

    def forward(self, x, attention_mask=None):
        x = x + self.self_attn(self.input_layernorm(x), attention_mask)
        return x + self.mlp(self.post_attention_layernorm(x))


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(LlamaDecoderLayer(cfg) for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, input_ids, attention_mask=None):
        x = self.embed_tokens(input_ids)
        if torch.is_autocast_enabled(x.device.type):
            x = x.to(torch.get_autocast_dtype(x.device.type))
        for layer in self.layers:
            x = layer(x, attention_mask)
        return self.norm(x)


class LlamaForCausalLM(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.config = cfg
        self.model = LlamaModel(cfg)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.apply(init_weights)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
            self.lm_head.weight._sb_tied = True     # two gradients per backward: layers must hand theirs to autograd

    def forward(self, input_ids, attention_mask=None, labels=None, **_):
        hidden = self.model(input_ids, attention_mask)
        if labels is not None and self.config.loss_chunk:
            return ModelOutput(loss=lm_loss(hidden, labels, self.lm_head, self.config.loss_chunk))
        logits = self.lm_head(hidden)
        return ModelOutput(loss=lm_loss(logits, labels) if labels is not None else None, logits=logits)
