"""LoRA and full training memory; BERT labels are synthetic.

Grid ``lora`` (deployment; 12 cells).  Parity: experiments/benchmarks/lora.py.

    python -m experiments.benchmarks.lora --dry-run
    python -m experiments.benchmarks.lora --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry

NAME = "lora"


def cells():
    return _entry.cells(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
