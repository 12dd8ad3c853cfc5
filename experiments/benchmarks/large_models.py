"""7B/8B context lengths, batches, and composed memory frontier.

Grid ``large_models`` (deployment; 12 cells).  Parity: experiments/benchmarks/large_models.py.

    python -m experiments.benchmarks.large_models --dry-run
    python -m experiments.benchmarks.large_models --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

NAME = "large_models"


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


from .probes import maxbatch, maxlen, one, sweep  # noqa: E402,F401  (search helpers bound to this grid's arms by the caller)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
