"""LoRA and full training memory; BERT labels are synthetic.

Grid ``lora`` (deployment; 12 cells).  Parity: experiments/benchmarks/lora.py.

    python -m experiments.benchmarks.lora --dry-run
    python -m experiments.benchmarks.lora --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "lora")


CFG = {"rank": 8, "residual_budget": 0.005, "residual_bits": 8, "surface": "mlp", "min_features": 256, "chunk_rows": 512}


def run_lora(model_id, bs, seq, steps, seed, use_lora, use_stacr, qlora=False, tag="", **run_kw):
    """One adapter-composition cell: rank-8 adapters on the attention projections and/or STAC-R on the *trainable* MLP inputs.

    With adapters the MLP is frozen, nothing there is saved for a weight gradient, and the compression surface is empty
    (``empty_compression_control`` in the row): the negative-composition control.
    """
    if qlora:
        raise ValueError("Use the qlora experiment for NF4 quantised bases")
    from . import common

    method = ("lora" if use_lora else "full") + ("+stacr" if use_stacr else "")
    rec = common.run_config(method, seed, model_id=model_id, bs=bs, seq=seq, steps=steps, measure_from=min(6, steps - 1), eval_batches=0,
                            stacr_cfg=dict(CFG, turbo_after_step=None) if use_stacr else None, lora=bool(use_lora), **run_kw)
    rec["tag"] = tag
    return rec


if __name__ == "__main__":
    raise SystemExit(main())
