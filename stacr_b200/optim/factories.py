"""Optimizer factories usable as ``optimizer: "stacr_b200.optim.factories:<name>"`` in a trainer config.

A factory receives ``(model, resolved_config)`` and returns a ``torch.optim.Optimizer``.
"""

from __future__ import annotations

import torch


def sgd(model, config):
    """Plain SGD (no momentum): handy for exact-arithmetic checks of the training loop."""
    params = [p for p in model.parameters() if p.requires_grad]
    return torch.optim.SGD(params, lr=float(config.get("lr", 1e-2)), weight_decay=float(config.get("weight_decay", 0.0)))


def adamw_bf16_shadow(model, config):
    """In-tree AdamW that also refreshes a bf16 shadow of every weight inside the update kernel."""
    from .adamw import AdamW

    params = [p for p in model.parameters() if p.requires_grad]
    return AdamW(params, lr=float(config.get("lr", 5e-5)), weight_decay=float(config.get("weight_decay", 0.0)), bf16_shadow=True)
