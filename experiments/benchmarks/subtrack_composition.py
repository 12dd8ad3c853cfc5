"""Upstream SubTrack++ BERT/SST-2 and adaptive STAC-R composition.

Grid ``subtrack_composition`` (comparators; 3 cells).  Parity: experiments/benchmarks/subtrack_composition.py.

    python -m experiments.benchmarks.subtrack_composition --dry-run
    python -m experiments.benchmarks.subtrack_composition --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

NAME = "subtrack_composition"


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
