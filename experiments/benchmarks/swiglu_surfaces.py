"""SwiGLU rank, token shape, and down-projection surface sweep.

Grid ``swiglu_surfaces`` (mechanism; 8 cells).  Parity: experiments/benchmarks/swiglu_surfaces.py.

    python -m experiments.benchmarks.swiglu_surfaces --dry-run
    python -m experiments.benchmarks.swiglu_surfaces --steps 20 --seeds 42
"""

from __future__ import annotations

from . import _entry
from .probes import complement  # noqa: F401

_entry.bind(globals(), "swiglu_surfaces")


def down_proj_names(model):
    """The SwiGLU down projections: the one MLP projection whose input has the expanded width."""
    return [n for n, m in model.named_modules() if n.endswith("down_proj") and getattr(getattr(m, "weight", None), "dim", lambda: 0)() == 2]


def cfg_for(model_id, surf_name, surf_cfg, rank):
    """Layer options for a named surface at a rank; keys starting with ``_`` are directives, ``_down_only`` pins the selection
    to the down projections (found on a CPU probe copy of the model)."""
    cfg = {"rank": rank, "residual_budget": 0.005, "residual_bits": 8, "chunk_rows": 512, **{k: v for k, v in surf_cfg.items() if not k.startswith("_")}}
    if surf_cfg.get("_down_only"):
        from . import common

        probe = common.load_model(model_id, "cpu")
        cfg["surface"], cfg["extra_names"] = "none", down_proj_names(probe)
        del probe
    return cfg


if __name__ == "__main__":
    raise SystemExit(main())
