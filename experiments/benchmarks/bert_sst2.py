"""BERT classification accuracy with full compression and Turbo-fast.

Grid ``bert_sst2`` (quality; 3 cells).  Parity: experiments/benchmarks/bert_sst2.py.

    python -m experiments.benchmarks.bert_sst2 --dry-run
    python -m experiments.benchmarks.bert_sst2 --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "bert_sst2")


def sst2(method="baseline", stacr_cfg=None, bs=32, seq=128, steps=60, seed=42, **run_kw):
    """One BERT sequence-classification cell (random class labels offline: a memory/throughput protocol)."""
    from . import common

    return common.run_config(method, seed, model_id="bert-base-uncased", bs=bs, seq=seq, steps=steps, stacr_cfg=stacr_cfg, **run_kw)


if __name__ == "__main__":
    raise SystemExit(main())
