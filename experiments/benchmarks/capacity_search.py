"""Ascending batch search to the first allocation failure.

Grid ``capacity_search`` (deployment; 16 cells).  Parity: experiments/benchmarks/capacity_search.py.

    python -m experiments.benchmarks.capacity_search --dry-run
    python -m experiments.benchmarks.capacity_search --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "capacity_search")


def largest_fitting(model_id, seq, dtype, lo, hi, method, cfg, out=None, tag="capacity", **run_kw):
    """The largest batch in ``lo..hi`` that trains; see :func:`probes.largest_fitting`."""
    from . import probes

    return probes.largest_fitting(model_id, seq, dtype, lo, hi, method, cfg, out, tag, **run_kw)


if __name__ == "__main__":
    raise SystemExit(main())
