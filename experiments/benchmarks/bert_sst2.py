"""BERT classification accuracy with full compression and Turbo-fast.

Grid ``bert_sst2`` (quality; 3 cells).  Parity: experiments/benchmarks/bert_sst2.py.

    python -m experiments.benchmarks.bert_sst2 --dry-run
    python -m experiments.benchmarks.bert_sst2 --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

NAME = "bert_sst2"


def cells():
    return _entry.cells(NAME)


def rows():
    return _entry.cells(NAME)


def arms():
    return _entry.arms(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def run_cohort(selector, seeds=(42,), output=None):
    return _entry.run_cohort(NAME, selector, seeds, output)


def sst2(method="baseline", stacr_cfg=None, bs=32, seq=128, steps=60, seed=42, **run_kw):
    """One BERT sequence-classification cell (random class labels offline: a memory/throughput protocol)."""
    from . import common

    return common.run_config(method, seed, model_id="bert-base-uncased", bs=bs, seq=seq, steps=steps, stacr_cfg=stacr_cfg, **run_kw)


def one(method, seed=42, **overrides):
    return _entry.one(NAME, method, seed, **overrides)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
