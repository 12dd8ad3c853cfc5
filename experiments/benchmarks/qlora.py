"""NF4 QLoRA memory and supported composition; synthetic BERT labels.

Grid ``qlora`` (deployment; 6 cells).  Parity: experiments/benchmarks/qlora.py.

    python -m experiments.benchmarks.qlora --dry-run
    python -m experiments.benchmarks.qlora --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry

NAME = "qlora"


def cells():
    return _entry.cells(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
