"""Eager, SDPA, and FlashAttention at the same saved surface.

Grid ``attention_kernels`` (systems; 9 cells).  Parity: experiments/benchmarks/attention_kernels.py.

    python -m experiments.benchmarks.attention_kernels --dry-run
    python -m experiments.benchmarks.attention_kernels --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

NAME = "attention_kernels"


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
