"""STAC-R, Oja-only, OASIS, PRAC, and random basis controls.

Grid ``basis_comparison`` (quality; 6 cells).  Parity: experiments/benchmarks/basis_comparison.py.

    python -m experiments.benchmarks.basis_comparison --dry-run
    python -m experiments.benchmarks.basis_comparison --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

NAME = "basis_comparison"


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


def one(method, seed=42, **overrides):
    return _entry.one(NAME, method, seed, **overrides)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
