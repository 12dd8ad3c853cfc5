"""Allocated, reserved, and NVML memory over 600 steps.

Grid ``allocator_stability`` (systems; 3 cells).  Parity: experiments/benchmarks/allocator_stability.py.

    python -m experiments.benchmarks.allocator_stability --dry-run
    python -m experiments.benchmarks.allocator_stability --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "allocator_stability")


def trace(method, cfg, model_id="qwen2.5-1.5b", bs=2, seq=1024, steps=600, **run_kw):
    """A long run with allocated / reserved / NVML memory read at steps 10, 50, 100, 200, ... and the last one.

    Flat curves mean the compressed layers' transient buffers do not fragment the caching allocator over time.
    """
    from . import common

    return common.run_config(method, 42, model_id=model_id, bs=bs, seq=seq, steps=steps, measure_from=0, eval_batches=0,
                             stacr_cfg=dict(cfg, turbo_after_step=None) if cfg else None, trace_memory=True, **run_kw)


if __name__ == "__main__":
    raise SystemExit(main())
