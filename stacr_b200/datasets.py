"""Training examples: synthetic token streams (no network needed) and Hugging Face text sets.

``build_examples`` follows stacr/datasets.py:16-143 of the reference project (sst2, mrpc,
wikitext, openwebtext, plain text files, packed fixed-length blocks) and adds
``dataset: synthetic``: uniform-random token ids from a seed, next-token labels for language
modelling or Bernoulli(0.5) labels for sequence classification.
"""

from __future__ import annotations

from typing import Any

import torch

_ALIASES = {
    "wikitext": [("wikitext", "wikitext-103-raw-v1"), ("Salesforce/wikitext", "wikitext-103-raw-v1")],
    "wikitext-103": [("wikitext", "wikitext-103-raw-v1"), ("Salesforce/wikitext", "wikitext-103-raw-v1")],
    "wikitext-2": [("wikitext", "wikitext-2-raw-v1"), ("Salesforce/wikitext", "wikitext-2-raw-v1")],
    "openwebtext": [("Skylion007/openwebtext", None), ("openwebtext", None)],
    "sst2": [("glue", "sst2"), ("nyu-mll/glue", "sst2")],
    "mrpc": [("glue", "mrpc"), ("nyu-mll/glue", "mrpc")],
}


def load_hf_dataset(name: str, split: str, revision: str | None = None):
    """Try each known hub alias of ``name`` in turn; raise the last error when none resolves."""
    from datasets import load_dataset

    last: Exception | None = None
    for repo, subset in _ALIASES.get(name, [(name, None)]):
        try:
            return load_dataset(repo, subset, split=split, revision=revision)
        except Exception as exc:  # noqa: BLE001 - alias fallbacks
            last = exc
    raise RuntimeError(f"Could not load dataset {name!r}") from last


def synthetic_token_examples(count: int, seq_len: int, vocab_size: int, seed: int, task: str = "language_modeling") -> list[dict]:
    gen = torch.Generator().manual_seed(int(seed))
    ids = torch.randint(0, int(vocab_size), (int(count), int(seq_len)), generator=gen)
    out = []
    for row in ids:
        ex: dict[str, Any] = {"input_ids": row, "attention_mask": torch.ones_like(row)}
        if task == "sequence_classification":
            ex["labels"] = torch.bernoulli(torch.tensor(0.5), generator=gen).long()
        else:
            ex["labels"] = row.clone()
        out.append(ex)
    return out


def tokenize_text_dataset(dataset, tokenizer, text_key: str, max_length: int):
    """Fixed-length tokenisation of a ``datasets`` table (truncate and pad to ``max_length``); the text columns are dropped."""
    def encode(batch):
        return tokenizer(batch[text_key], truncation=True, padding="max_length", max_length=max_length)

    return dataset.map(encode, batched=True, remove_columns=dataset.column_names)


def packed_text_blocks(texts, tokenizer, seq_len: int, max_examples: int | None = None) -> list[dict]:
    """Concatenate tokenised documents (EOS-separated) and cut fixed ``seq_len`` blocks."""
    eos = tokenizer.eos_token_id
    stream: list[int] = []
    blocks: list[dict] = []
    for text in texts:
        if not text or not text.strip():
            continue
        stream.extend(tokenizer(text)["input_ids"])
        if eos is not None:
            stream.append(eos)
        while len(stream) >= seq_len:
            chunk = torch.tensor(stream[:seq_len], dtype=torch.long)
            del stream[:seq_len]
            blocks.append({"input_ids": chunk, "attention_mask": torch.ones_like(chunk), "labels": chunk.clone()})
            if max_examples and len(blocks) >= max_examples:
                return blocks
    return blocks


def build_examples(config: dict, tokenizer, validation: bool = False) -> list[dict]:
    name = str(config.get("dataset", "synthetic"))
    task = config.get("task", "language_modeling")
    seq_len = int(config.get("seq_len", 128))
    limit = int(config.get("max_eval_examples" if validation else "max_examples", 64 if validation else 1024))
    if name == "synthetic":
        vocab = int(config.get("vocab_size", getattr(tokenizer, "vocab_size", 1024) if tokenizer else 1024))
        return synthetic_token_examples(limit, seq_len, vocab, int(config.get("seed", 42)) + (1 if validation else 0), task)
    if name == "text":
        path = config.get("validation_file" if validation else "train_file")
        if not path:
            raise ValueError("dataset=text needs train_file/validation_file")
        with open(path, "r", encoding="utf-8") as fh:
            return packed_text_blocks(fh, tokenizer, seq_len, limit)
    split = "validation" if validation else "train"
    data = load_hf_dataset(name, split, config.get("dataset_revision"))
    if name in ("sst2", "mrpc"):
        rows = []
        for ex in data.select(range(min(limit, len(data)))):
            first = ex["sentence"] if name == "sst2" else ex["sentence1"]
            second = None if name == "sst2" else ex["sentence2"]
            enc = tokenizer(first, second, truncation=True, max_length=seq_len, padding="max_length", return_tensors="pt")
            rows.append({"input_ids": enc["input_ids"][0], "attention_mask": enc["attention_mask"][0], "labels": torch.tensor(int(ex["label"]))})
        return rows
    return packed_text_blocks((ex["text"] for ex in data), tokenizer, seq_len, limit)
