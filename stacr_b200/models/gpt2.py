"""GPT-2 family decoder (learned positions, pre-LN, tanh-GELU MLP, tied LM head)."""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from .common import causal_attention, Embedding, GELU, init_weights, LayerNorm, Linear, lm_loss, ModelOutput


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: int | None = None
    layer_norm_epsilon: float = 1e-5
    resid_pdrop: float = 0.0
    embd_pdrop: float = 0.0
    attn_pdrop: float = 0.0
    tie_word_embeddings: bool = True
    loss_chunk: int = 0

    @property
    def inner(self) -> int:
        return self.n_inner or 4 * self.n_embd


PRESETS = {
    "gpt2": dict(n_embd=768, n_layer=12, n_head=12),
    "gpt2-medium": dict(n_embd=1024, n_layer=24, n_head=16),
    "gpt2-large": dict(n_embd=1280, n_layer=36, n_head=20),
    "gpt2-xl": dict(n_embd=1600, n_layer=48, n_head=25),
    # CPU smoke shape: 4 layers, d 256, 4 heads, MLP 1024, vocab 1024
    "gpt-tiny": dict(n_embd=256, n_layer=4, n_head=4, vocab_size=1024, n_positions=128),
}


class GPT2Attention(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.n_head, self.head_dim = cfg.n_head, cfg.n_embd // cfg.n_head
        self.c_attn = Linear(cfg.n_embd, 3 * cfg.n_embd)
        self.c_proj = Linear(cfg.n_embd, cfg.n_embd)
        self.attn_pdrop = cfg.attn_pdrop
        self.resid_dropout = nn.Dropout(cfg.resid_pdrop)

    def forward(self, x, attention_mask=None):
        b, s, d = x.shape
        qkv = self.c_attn(x).view(b, s, 3, self.n_head, self.head_dim)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        ctx = causal_attention(q, k, v, causal=True, attention_mask=attention_mask, dropout_p=self.attn_pdrop, training=self.training)
        return self.resid_dropout(self.c_proj(ctx.transpose(1, 2).reshape(b, s, d)))


class GPT2MLP(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.c_fc = Linear(cfg.n_embd, cfg.inner)
        self.act = GELU("tanh")
        self.c_proj = Linear(cfg.inner, cfg.n_embd)
        self.dropout = nn.Dropout(cfg.resid_pdrop)

    def forward(self, x):
        return self.dropout(self.c_proj(self.act(self.c_fc(x))))


class GPT2Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.ln_1 = LayerNorm(cfg.n_embd, eps=cfg.layer_norm_epsilon)
        self.attn = GPT2Attention(cfg)
        self.ln_2 = LayerNorm(cfg.n_embd, eps=cfg.layer_norm_epsilon)
        self.mlp = GPT2MLP(cfg)

    def forward(self, x, attention_mask=None):
        x = x + self.attn(self.ln_1(x), attention_mask)
        return x + self.mlp(self.ln_2(x))


class GPT2Model(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.wte = Embedding(cfg.vocab_size, cfg.n_embd)
        self.wpe = Embedding(cfg.n_positions, cfg.n_embd)
        self.drop = nn.Dropout(cfg.embd_pdrop)
        self.h = nn.ModuleList(GPT2Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = LayerNorm(cfg.n_embd, eps=cfg.layer_norm_epsilon)

    def forward(self, input_ids, attention_mask=None):
        pos = torch.arange(input_ids.shape[1], device=input_ids.device)
        x = self.drop(self.wte(input_ids) + self.wpe(pos))
        if torch.is_autocast_enabled(x.device.type):
            x = x.to(torch.get_autocast_dtype(x.device.type))
        for block in self.h:
            x = block(x, attention_mask)
        return self.ln_f(x)


class GPT2LMHeadModel(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.config = cfg
        self.transformer = GPT2Model(cfg)
        self.lm_head = Linear(cfg.n_embd, cfg.vocab_size, bias=False)
        self.apply(init_weights)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / (2 * cfg.n_layer) ** 0.5)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.transformer.wte.weight
            self.lm_head.weight._sb_tied = True     # two gradients per backward: layers must hand theirs to autograd

    def forward(self, input_ids, attention_mask=None, labels=None, **_):
        hidden = self.transformer(input_ids, attention_mask)
        # training on a GPU with the stock 50257-entry vocabulary: the head and the loss run together on a padded logits
        # buffer (an odd leading dimension would push the library onto unaligned GEMM kernels); no logits are returned
        fused_head = self.training and hidden.is_cuda and self.config.vocab_size % 8 != 0 and torch.is_autocast_enabled()
        if labels is not None and (self.config.loss_chunk or fused_head):
            return ModelOutput(loss=lm_loss(hidden, labels, self.lm_head, self.config.loss_chunk))
        logits = self.lm_head(hidden)
        loss = lm_loss(logits, labels) if labels is not None else None
        return ModelOutput(loss=loss, logits=logits)
