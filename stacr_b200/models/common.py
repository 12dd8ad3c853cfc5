"""Shared building blocks of the in-tree model zoo.

The models are defined from a config (random init, no downloads) and name their submodules as
the Hugging Face implementations do (``transformer.h.N.mlp.c_fc``,
``gpt_neox.layers.N.mlp.dense_h_to_4h``, ``bert.encoder.layer.N.intermediate.dense``) so that
surface classification, block discovery and checkpoints line up with what users of the
reference expect.  Hot element-wise/normalisation ops go through ``stacr_b200.ops.nn_ops``,
which runs the sm_100a kernels for bf16 CUDA tensors.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn
from torch.nn import functional as F

from ..ops import attention as attention_ops
from ..ops import nn_ops


@dataclass
class ModelOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None

    def __getitem__(self, key):
        return getattr(self, key)


class LayerNorm(nn.LayerNorm):
    """LayerNorm whose bf16 CUDA path is the fused kernel (fp32 statistics, bf16 in/out)."""

    def forward(self, x):
        return nn_ops.layer_norm(x, self.weight, self.bias, self.eps)


class Linear(nn.Linear):
    """``nn.Linear`` (same parameters, same state-dict keys) whose training path on a B200 forms the weight gradient in
    fp32 directly (see ``ops.nn_ops.linear``); everywhere else it is the stock layer."""

    def forward(self, x):
        return nn_ops.linear(x, self.weight, self.bias)


class Embedding(nn.Embedding):
    """``nn.Embedding`` (same parameter, same state-dict key) whose bf16-autocast path on a B200 is the in-tree lookup and
    scatter-add (see ``ops.nn_ops.embedding``); the output is then already in the autocast dtype."""

    def forward(self, ids):
        if self.max_norm is None and not self.sparse and not self.scale_grad_by_freq:
            return nn_ops.embedding(ids, self.weight, self.padding_idx)
        return super().forward(ids)


class GELU(nn.Module):
    def __init__(self, approximate: str = "none"):
        super().__init__()
        self.approximate = approximate

    def forward(self, x):
        return nn_ops.gelu(x, self.approximate)


def _attention_engine() -> str:
    """``STACR_ATTENTION``: ``library`` (default: the fused attention ``torch`` dispatches to, which measured faster on
    B200) or ``intree`` (the tcgen05 kernels of ``ops/attention.py``: forward for gradient-free passes of every model,
    forward + backward on the fused QKV projection for the GPT-NeoX family at head_dim 128)."""
    return os.environ.get("STACR_ATTENTION", "library")


def causal_attention(q, k, v, *, causal: bool, attention_mask=None, dropout_p: float = 0.0, training: bool = False):
    """Softmax attention on ``[B, H, S, D]`` tensors (no ``S x S`` score tensor).

    A padding mask ``[B, S]`` (1 = keep) is turned into an additive bias only when it actually masks something.  With
    ``STACR_ATTENTION=intree`` and no gradient to record (evaluation, generation, recomputation-free inference) the
    in-tree kernel runs instead: it reads strided views of a fused QKV projection in place.
    """
    if (_attention_engine() == "intree" and not (torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad))
            and not (training and dropout_p > 0.0) and attention_ops.supported(q, k, v)):
        b, h, s, d = q.shape
        out, _ = attention_ops.forward(q, k, v, causal=causal, key_mask=attention_mask, need_lse=False)
        return out.view(b, s, h, d).transpose(1, 2)
    bias = None
    if attention_mask is not None and not bool(attention_mask.all()):
        keep = attention_mask[:, None, None, :].to(torch.bool)
        if causal:
            s = q.shape[-2]
            keep = keep & torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
            causal = False
        bias = keep
    return F.scaled_dot_product_attention(q, k, v, attn_mask=bias, dropout_p=dropout_p if training else 0.0, is_causal=causal and bias is None)


def lm_loss(logits_or_hidden, labels, lm_head: nn.Linear | None = None, chunk: int = 0):
    """Next-token cross-entropy with the usual shift; ``labels == -100`` are ignored."""
    if lm_head is not None:
        hidden = logits_or_hidden[:, :-1].reshape(-1, logits_or_hidden.shape[-1])
        target = labels[:, 1:].reshape(-1)
        return nn_ops.linear_cross_entropy(hidden, lm_head.weight, target, chunk=chunk)
    # every position is scored against the next token; the last one has none and is masked out, which keeps the
    # [B, S, V] logits as they are (slicing off the last position would copy the whole tensor, forward and backward)
    shifted = torch.cat((labels[:, 1:], labels.new_full((labels.shape[0], 1), -100)), dim=1)
    return nn_ops.cross_entropy(logits_or_hidden.reshape(-1, logits_or_hidden.shape[-1]), shifted.reshape(-1))


def init_weights(module: nn.Module, std: float = 0.02) -> None:
    if isinstance(module, nn.Linear):
        nn.init.normal_(module.weight, mean=0.0, std=std)
        if module.bias is not None:
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        nn.init.normal_(module.weight, mean=0.0, std=std)
    elif isinstance(module, nn.LayerNorm):
        nn.init.ones_(module.weight)
        nn.init.zeros_(module.bias)
