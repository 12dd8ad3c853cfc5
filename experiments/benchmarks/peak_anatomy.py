"""Training-phase allocation and chunked cross-entropy controls.

Grid ``peak_anatomy`` (mechanism; 4 cells).  Parity: experiments/benchmarks/peak_anatomy.py.

    python -m experiments.benchmarks.peak_anatomy --dry-run
    python -m experiments.benchmarks.peak_anatomy --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry

NAME = "peak_anatomy"


def cells():
    return _entry.cells(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
