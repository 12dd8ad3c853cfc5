"""Training-phase allocation and chunked cross-entropy controls.

Grid ``peak_anatomy`` (mechanism; 4 cells).  Parity: experiments/benchmarks/peak_anatomy.py.

    python -m experiments.benchmarks.peak_anatomy --dry-run
    python -m experiments.benchmarks.peak_anatomy --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "peak_anatomy")


def phase_run(method, cfg, model_id="gpt2-medium", bs=8, seq=1024, **run_kw):
    """One cell whose row carries ``phase_peaks_GiB``: the allocator peak after forward, backward and the optimizer step."""
    from . import common

    return common.run_config(method, 42, model_id=model_id, bs=bs, seq=seq, stacr_cfg=cfg, phase_profile=True, eval_batches=0, **run_kw)


def ce_run(chunk, model_id="gpt2-medium", bs=8, seq=1024, **run_kw):
    """The same with the language-model loss computed ``chunk`` tokens at a time, which removes the full logits from the peak."""
    from . import common

    return common.run_config(f"chunked_ce_{chunk}", 42, model_id=model_id, bs=bs, seq=seq, phase_profile=True, eval_batches=0,
                             model_overrides={**run_kw.pop("model_overrides", {}), "loss_chunk": int(chunk)}, **run_kw)


if __name__ == "__main__":
    raise SystemExit(main())
