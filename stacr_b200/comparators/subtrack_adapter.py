"""SubTrack-style optimizer factory (parity: comparators/subtrack_adapter.py:146-224 of the reference project).

The reference loads an external SubTrack++ source tree; here the in-tree ``SubTrackAdamW`` (projected Adam moments with
a Grassmannian-tracked subspace) is built from the same trainer keys.
"""

from __future__ import annotations


def subtrack_available() -> bool:
    return True


def create_subtrack_optimizer(model, config):
    from .lowrank_optim import SubTrackAdamW, split_param_groups

    groups = split_param_groups(
        model, config.get("subtrack_target_modules"), float(config.get("weight_decay", 0.0)),
        rank=int(config.get("subtrack_rank", 8)), update_proj_gap=int(config.get("subtrack_update_interval", 200)),
        scale=float(config.get("subtrack_scale", 0.25)), proj_type=config.get("subtrack_proj_type", "std"),
        step_size=float(config.get("subtrack_step_size", 0.1)), track_interval=max(1, int(config.get("subtrack_update_interval", 200)) // 20),
    )
    return SubTrackAdamW(groups, lr=float(config.get("lr", 5e-5)))
