"""Exact and compressed gradients using one model in memory.

Grid ``single_model_fidelity`` (fidelity; 2 cells).  Parity: experiments/benchmarks/single_model_fidelity.py.

    python -m experiments.benchmarks.single_model_fidelity --dry-run
    python -m experiments.benchmarks.single_model_fidelity --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

NAME = "single_model_fidelity"


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


from .probes import grads  # noqa: E402,F401  (paired gradients of one model, RNG seeded per call)


def one(method, seed=42, **overrides):
    return _entry.one(NAME, method, seed, **overrides)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
