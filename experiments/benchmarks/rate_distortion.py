"""Stored-byte and gradient-error frontier over rank and basis.

Grid ``rate_distortion`` (fidelity; 24 cells).  Parity: experiments/benchmarks/rate_distortion.py.

    python -m experiments.benchmarks.rate_distortion --dry-run
    python -m experiments.benchmarks.rate_distortion --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "rate_distortion")


def payload_bytes(kind, rank, budget, model_id="gpt2-medium", bs=4, seq=512, min_features=256, **overrides):
    """``(stored bytes, dense bytes, layers)`` of one batch's saved MLP inputs under a basis control at a rank and budget.

    Counts coefficients, residual and basis per wrapped layer for ``bs * seq`` rows of 2-byte activations; nothing is trained.
    """
    from stacr_b200.comparators.activation import apply_comparator

    from . import common

    model = common.load_model(model_id, "cpu", **overrides)
    layers = apply_comparator(model, kind, {"rank": rank, "residual_budget": budget, "surface": "mlp", "min_features": min_features})
    rows = bs * seq
    stored = sum(sum(v for k, v in layer.stored_bytes(rows, 2).items() if k in ("coeff", "residual", "basis")) for layer in layers)
    dense = sum(rows * layer.in_features * 2 for layer in layers)
    return stored, dense, len(layers)


if __name__ == "__main__":
    raise SystemExit(main())
