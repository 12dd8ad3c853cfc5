"""BERT classification accuracy with full compression and Turbo-fast.

Grid ``bert_sst2`` (quality; 3 cells).  Parity: experiments/benchmarks/bert_sst2.py.

    python -m experiments.benchmarks.bert_sst2 --dry-run
    python -m experiments.benchmarks.bert_sst2 --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry

NAME = "bert_sst2"


def cells():
    return _entry.cells(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
