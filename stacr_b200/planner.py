"""Toy per-layer planner (parity: stacr/planner.py:1-38 of the reference project)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class LayerPlan:
    name: str
    features: int
    rank: int
    residual_budget: float
    compress: bool


def choose_rank(features: int, requested_rank: int, min_rank: int = 1) -> int:
    return max(int(min_rank), min(int(requested_rank), int(features)))


def plan_linear_layers(named_modules, rank: int = 8, residual_budget: float = 0.005, min_features: int = 128):
    """One plan per module exposing ``in_features``; layers narrower than ``min_features`` stay dense."""
    plans = []
    for name, module in named_modules:
        width = getattr(module, "in_features", None)
        if width is None:
            continue
        width = int(width)
        plans.append(LayerPlan(name, width, choose_rank(width, rank), float(residual_budget), width >= int(min_features)))
    return plans
