"""BERT encoder with a pooled sequence-classification head (post-LN, learned positions, erf-GELU)."""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn
from torch.nn import functional as F

from .common import causal_attention, Embedding, GELU, init_weights, LayerNorm, Linear, ModelOutput


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_dropout_prob: float = 0.0
    attention_probs_dropout_prob: float = 0.0
    num_labels: int = 2


PRESETS = {
    "bert-base-uncased": dict(),
    "bert-base": dict(),
    "bert-large-uncased": dict(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096),
    "bert-tiny": dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=512, vocab_size=1024, max_position_embeddings=128),
}


class BertEmbeddings(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.word_embeddings = Embedding(cfg.vocab_size, cfg.hidden_size)
        self.position_embeddings = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size)
        self.token_type_embeddings = nn.Embedding(cfg.type_vocab_size, cfg.hidden_size)
        self.LayerNorm = LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.dropout = nn.Dropout(cfg.hidden_dropout_prob)

    def forward(self, input_ids, token_type_ids=None):
        pos = torch.arange(input_ids.shape[1], device=input_ids.device)
        tt = torch.zeros_like(input_ids) if token_type_ids is None else token_type_ids
        x = self.word_embeddings(input_ids) + self.position_embeddings(pos) + self.token_type_embeddings(tt)
        if torch.is_autocast_enabled(x.device.type):
            x = x.to(torch.get_autocast_dtype(x.device.type))
        return self.dropout(self.LayerNorm(x))


class BertSelfAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.n_head, self.head_dim = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads
        self.query = Linear(cfg.hidden_size, cfg.hidden_size)
        self.key = Linear(cfg.hidden_size, cfg.hidden_size)
        self.value = Linear(cfg.hidden_size, cfg.hidden_size)
        self.p = cfg.attention_probs_dropout_prob

    def forward(self, x, attention_mask=None):
        b, s, d = x.shape
        split = lambda t: t.view(b, s, self.n_head, self.head_dim).transpose(1, 2)
        ctx = causal_attention(split(self.query(x)), split(self.key(x)), split(self.value(x)), causal=False,
                               attention_mask=attention_mask, dropout_p=self.p, training=self.training)
        return ctx.transpose(1, 2).reshape(b, s, d)


class BertSelfOutput(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.dense = Linear(cfg.hidden_size, cfg.hidden_size)
        self.LayerNorm = LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.dropout = nn.Dropout(cfg.hidden_dropout_prob)

    def forward(self, h, residual):
        return self.LayerNorm(self.dropout(self.dense(h)) + residual)


class BertAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.self = BertSelfAttention(cfg)
        self.output = BertSelfOutput(cfg)

    def forward(self, x, attention_mask=None):
        return self.output(self.self(x, attention_mask), x)


class BertIntermediate(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.dense = Linear(cfg.hidden_size, cfg.intermediate_size)
        self.intermediate_act_fn = GELU("none")

    def forward(self, x):
        return self.intermediate_act_fn(self.dense(x))


class BertOutput(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.dense = Linear(cfg.intermediate_size, cfg.hidden_size)
        self.LayerNorm = LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.dropout = nn.Dropout(cfg.hidden_dropout_prob)

    def forward(self, h, residual):
        return self.LayerNorm(self.dropout(self.dense(h)) + residual)


class BertLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.attention = BertAttention(cfg)
        self.intermediate = BertIntermediate(cfg)
        self.output = BertOutput(cfg)

    def forward(self, x, attention_mask=None):
        a = self.attention(x, attention_mask)
        return self.output(self.intermediate(a), a)


class BertEncoder(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.layer = nn.ModuleList(BertLayer(cfg) for _ in range(cfg.num_hidden_layers))

    def forward(self, x, attention_mask=None):
        for layer in self.layer:
            x = layer(x, attention_mask)
        return x


class BertPooler(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.dense = Linear(cfg.hidden_size, cfg.hidden_size)

    def forward(self, x):
        return torch.tanh(self.dense(x[:, 0]))


class BertModel(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.embeddings = BertEmbeddings(cfg)
        self.encoder = BertEncoder(cfg)
        self.pooler = BertPooler(cfg)

    def forward(self, input_ids, attention_mask=None, token_type_ids=None):
        x = self.encoder(self.embeddings(input_ids, token_type_ids), attention_mask)
        return x, self.pooler(x)


class BertForSequenceClassification(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.config = cfg
        self.bert = BertModel(cfg)
        self.dropout = nn.Dropout(cfg.hidden_dropout_prob)
        self.classifier = Linear(cfg.hidden_size, cfg.num_labels)
        self.apply(init_weights)

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, labels=None, **_):
        _, pooled = self.bert(input_ids, attention_mask, token_type_ids)
        logits = self.classifier(self.dropout(pooled))
        loss = F.cross_entropy(logits.float(), labels) if labels is not None else None
        return ModelOutput(loss=loss, logits=logits)
