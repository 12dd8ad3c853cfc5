"""Data for the INSTANT scripts (parity: comparators/instant/dataset_prep.py).

WikiText-103 and GLUE come from the local Hugging Face cache when present; with no cache (or ``synthetic=True``)
the loaders return random token blocks of the same shapes so that the scripts run end to end anywhere.
"""

from __future__ import annotations

import math

import torch

from ...datasets import load_hf_dataset, packed_text_blocks, synthetic_token_examples


def load_wikitext103(tokenizer=None, max_length: int = 512, *, synthetic: bool = False, vocab_size: int = 50257,
                     train_examples: int = 64, val_examples: int = 16, seed: int = 0):
    """``(train, validation)`` lists of ``{"input_ids", "labels"}`` blocks of ``max_length`` tokens."""
    if not synthetic and tokenizer is not None:
        try:
            train = load_hf_dataset("wikitext-103-raw-v1", "train")
            val = load_hf_dataset("wikitext-103-raw-v1", "validation")
            return (packed_text_blocks((r["text"] for r in train), tokenizer, max_length),
                    packed_text_blocks((r["text"] for r in val), tokenizer, max_length))
        except Exception:
            pass
    return (synthetic_token_examples(train_examples, max_length, vocab_size, seed),
            synthetic_token_examples(val_examples, max_length, vocab_size, seed + 1))


def load_classification(task: str = "sst2", tokenizer=None, max_length: int = 128, *, vocab_size: int = 30522,
                        train_examples: int = 64, val_examples: int = 32, seed: int = 0):
    """Synthetic two-class token blocks with the shapes of a GLUE task."""
    return (synthetic_token_examples(train_examples, max_length, vocab_size, seed, task="sequence_classification"),
            synthetic_token_examples(val_examples, max_length, vocab_size, seed + 1, task="sequence_classification"))


def compute_perplexity(eval_pred) -> dict:
    """``{"perplexity": exp(mean next-token loss)}`` from ``(logits, labels)``."""
    logits, labels = eval_pred
    logits, labels = torch.as_tensor(logits).float(), torch.as_tensor(labels).long()
    loss = torch.nn.functional.cross_entropy(logits[..., :-1, :].reshape(-1, logits.shape[-1]), labels[..., 1:].reshape(-1),
                                             ignore_index=-100)
    return {"perplexity": math.exp(min(float(loss), 50.0))}


def compute_metrics_with_args(args):
    """Accuracy metric closure for the classification script."""
    def compute(eval_pred):
        logits, labels = eval_pred
        pred = torch.as_tensor(logits).argmax(-1)
        return {"accuracy": float((pred == torch.as_tensor(labels)).float().mean())}
    return compute
