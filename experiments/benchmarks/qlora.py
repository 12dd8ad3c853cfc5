"""NF4 QLoRA memory and supported composition; synthetic BERT labels.

Grid ``qlora`` (deployment; 6 cells).  Parity: experiments/benchmarks/qlora.py.

    python -m experiments.benchmarks.qlora --dry-run
    python -m experiments.benchmarks.qlora --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "qlora")


CFG = {"rank": 8, "residual_budget": 0.005, "residual_bits": 8, "surface": "mlp", "min_features": 256, "chunk_rows": 512}
MODEL = "bert-base-uncased"


def build(kind: str, model_id: str = MODEL, device: str = "cuda", **overrides):
    """``full``: the plain classifier; ``lora``: rank-8 adapters on query/value over a frozen fp32 base; ``qlora``: the same
    adapters over a base quantised to 4-bit NormalFloat with double-quantised scales."""
    from stacr_b200.protocols.lora import apply_lora

    from . import common

    if kind not in ("full", "lora", "qlora"):
        raise ValueError(f"unknown kind {kind!r}")
    model = common.load_model(model_id, device, **overrides)
    if kind != "full":
        apply_lora(model, r=8, alpha=16.0, quantize_base=kind == "qlora")
    return model


def run_qlora(kind, use_stacr, bs, seq, steps, seed, tag="", model_id=MODEL, **run_kw):
    from . import common

    rec = common.run_config(kind + ("+stacr" if use_stacr else ""), seed, model_id=model_id, bs=bs, seq=seq, steps=steps, measure_from=min(6, steps - 1),
                            eval_batches=0, stacr_cfg=dict(CFG) if use_stacr else None, lora=kind == "lora", qlora=kind == "qlora", **run_kw)
    rec.update(tag=tag, quant=kind == "qlora")
    return rec


if __name__ == "__main__":
    raise SystemExit(main())
