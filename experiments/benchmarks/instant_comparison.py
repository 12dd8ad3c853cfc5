"""INSTANT SST-2, MRPC, and GPT-2 protocols with calibration.

Grid ``instant_comparison`` (comparators; 9 cells).  Parity: experiments/benchmarks/instant_comparison.py.

    python -m experiments.benchmarks.instant_comparison --dry-run
    python -m experiments.benchmarks.instant_comparison --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

NAME = "instant_comparison"


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


def enumerate_cells():
    """The grid's cells in run order (same as :func:`cells`)."""
    return cells()


def one(method, seed=42, **overrides):
    return _entry.one(NAME, method, seed, **overrides)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
