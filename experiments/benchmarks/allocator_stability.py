"""Allocated, reserved, and NVML memory over 600 steps.

Grid ``allocator_stability`` (systems; 3 cells).  Parity: experiments/benchmarks/allocator_stability.py.

    python -m experiments.benchmarks.allocator_stability --dry-run
    python -m experiments.benchmarks.allocator_stability --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry

NAME = "allocator_stability"


def cells():
    return _entry.cells(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
