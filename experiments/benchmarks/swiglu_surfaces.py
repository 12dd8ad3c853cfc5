"""SwiGLU rank, token shape, and down-projection surface sweep.

Grid ``swiglu_surfaces`` (mechanism; 8 cells).  Parity: experiments/benchmarks/swiglu_surfaces.py.

    python -m experiments.benchmarks.swiglu_surfaces --dry-run
    python -m experiments.benchmarks.swiglu_surfaces --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry

NAME = "swiglu_surfaces"


def cells():
    return _entry.cells(NAME)


def run(seeds=(42,), output=None):
    return _entry.run(NAME, seeds, output)


def main(argv=None) -> int:
    return _entry.main(NAME, argv)


if __name__ == "__main__":
    raise SystemExit(main())
