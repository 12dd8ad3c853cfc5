"""Model zoo (random init from a config) and the loader used by the trainer.

``load_model_and_tokenizer`` mirrors stacr/models.py:1-28 of the reference project: it returns
``(model, tokenizer)``.  In-tree architectures are built directly; any other name is delegated
to Hugging Face ``Auto*`` classes when ``transformers`` can resolve it locally.
"""

from __future__ import annotations

import torch

from . import bert, gpt2, llama, neox
from .bert import BertConfig, BertForSequenceClassification
from .common import ModelOutput
from .gpt2 import GPT2Config, GPT2LMHeadModel
from .llama import LlamaConfig, LlamaForCausalLM
from .neox import GPTNeoXForCausalLM, NeoXConfig

__all__ = [
    "BertConfig", "BertForSequenceClassification", "GPT2Config", "GPT2LMHeadModel", "GPTNeoXForCausalLM", "NeoXConfig",
    "LlamaConfig", "LlamaForCausalLM", "ModelOutput", "build_model", "load_model_and_tokenizer",
]


def _short(name: str) -> str:
    return name.split("/")[-1].lower()


def build_model(name: str, task: str = "language_modeling", **overrides):
    """Random-init in-tree model by preset name (``gpt2-medium``, ``pythia-1.4b``, ``bert-base-uncased``, ...)."""
    key = _short(name)
    if key in gpt2.PRESETS:
        return GPT2LMHeadModel(GPT2Config(**{**gpt2.PRESETS[key], **overrides}))
    if key in neox.PRESETS:
        return GPTNeoXForCausalLM(NeoXConfig(**{**neox.PRESETS[key], **overrides}))
    if key in llama.PRESETS:
        return LlamaForCausalLM(LlamaConfig(**{**llama.PRESETS[key], **overrides}))
    if key in bert.PRESETS:
        return BertForSequenceClassification(BertConfig(**{**bert.PRESETS[key], **overrides}))
    raise KeyError(f"No in-tree architecture for {name!r}")


def load_model_and_tokenizer(model_name, task="language_modeling", *, revision=None, attn_implementation=None,
                             dtype=torch.float32, local_files_only=False, random_init=False):
    """Return ``(model, tokenizer)``; falls back to in-tree random init when weights are not available."""
    if not random_init:
        try:
            from transformers import AutoModelForCausalLM, AutoModelForSequenceClassification, AutoTokenizer

            cls = AutoModelForSequenceClassification if task == "sequence_classification" else AutoModelForCausalLM
            kwargs = dict(revision=revision, local_files_only=local_files_only, torch_dtype=dtype)
            if attn_implementation:
                kwargs["attn_implementation"] = attn_implementation
            tok = AutoTokenizer.from_pretrained(model_name, revision=revision, local_files_only=local_files_only)
            if tok.pad_token is None:
                tok.pad_token = tok.eos_token
            return cls.from_pretrained(model_name, **kwargs), tok
        except Exception:
            pass
    return build_model(model_name, task).to(dtype), None
