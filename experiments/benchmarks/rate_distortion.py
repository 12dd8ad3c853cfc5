"""Stored-byte and gradient-error frontier over rank and basis.

Grid ``rate_distortion`` (fidelity; 24 cells).  Parity: experiments/benchmarks/rate_distortion.py.

    python -m experiments.benchmarks.rate_distortion --dry-run
    python -m experiments.benchmarks.rate_distortion --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry

NAME = "rate_distortion"


def cells():
    return _entry.cells(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
