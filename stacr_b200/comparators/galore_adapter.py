"""GaLore optimizer factory (parity: comparators/galore_adapter.py of the reference project).

Uses the ``galore_torch`` package when it is installed and the in-tree ``GaLoreAdamW`` otherwise, so the ``galore``
methods of the trainer run offline.
"""

from __future__ import annotations


def galore_available() -> bool:
    try:
        import galore_torch  # noqa: F401

        return True
    except Exception:
        return False


def create_galore_optimizer(model, lr=0.01, rank=128, update_proj_gap=200, scale=0.25, proj_type="std", weight_decay=0.0,
                            target_modules=None, prefer_external: bool = False):
    from .lowrank_optim import GaLoreAdamW, split_param_groups

    groups = split_param_groups(model, target_modules, weight_decay, rank=int(rank), update_proj_gap=int(update_proj_gap),
                                scale=float(scale), proj_type=proj_type)
    if prefer_external and galore_available():
        from galore_torch import GaLoreAdamW as External

        return External(groups, lr=lr)
    return GaLoreAdamW(groups, lr=lr)
