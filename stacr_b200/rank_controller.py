"""Host-side controllers for the *active prefix rank* of a tracked basis.

The basis buffer keeps its allocated width; a controller only decides how many leading columns a
forward uses, so rank can change at safe boundaries without resizing buffers.  API parity:
stacr/rank_controller.py:15-210 of the reference project.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, Mapping, Optional


@dataclass(frozen=True)
class RankDecision:
    active_rank: int
    reason_code: str
    changed: bool
    metric_value: Optional[float] = None


def _bounded(rank: int, lo: int, hi: int, available: int) -> int:
    lo = max(1, int(lo))
    hi = max(lo, int(hi))
    return min(max(1, int(available)), max(lo, min(int(rank), hi)))


def _decide(target: int, current: int, grow: str, shrink: str, keep: str, metric) -> RankDecision:
    code = grow if target > current else shrink if target < current else keep
    return RankDecision(target, code, target != current, metric)


def should_adjust_rank(schedule_step: int, last_adjust_step: int, adjust_interval: int) -> bool:
    """Rate-limit rank changes: true on the first call and every ``adjust_interval`` steps after."""
    if last_adjust_step < 0:
        return True
    return int(schedule_step) - int(last_adjust_step) >= max(1, int(adjust_interval))


def choose_variance_rank(
    coeff_energy_by_rank: Optional[Iterable[float]],
    current_rank: int,
    rank_min: int,
    rank_max: int,
    max_available_rank: int,
    variance_threshold: float,
) -> RankDecision:
    """Smallest prefix whose coefficient energy reaches ``variance_threshold`` of the total."""
    current = _bounded(current_rank, rank_min, rank_max, max_available_rank)
    if coeff_energy_by_rank is None:
        return RankDecision(current, "variance_cold_start", False, None)
    energy = []
    for raw in coeff_energy_by_rank:
        value = float(raw)
        if not math.isfinite(value):
            raise ValueError(f"Invalid coefficient energy: {raw!r}")
        energy.append(max(0.0, value))
    if not energy:
        return RankDecision(current, "variance_empty", False, 0.0)
    energy = energy[:max_available_rank]
    total = float(sum(energy))
    if total <= 0.0:
        floor = _bounded(rank_min, rank_min, rank_max, max_available_rank)
        return RankDecision(floor, "variance_zero_energy", floor != current, 0.0)
    goal = total * min(max(float(variance_threshold), 0.0), 1.0)
    acc, prefix = 0.0, 1
    for prefix, value in enumerate(energy, start=1):
        acc += value
        if acc >= goal:
            break
    target = _bounded(prefix, rank_min, rank_max, max_available_rank)
    return _decide(target, current, "variance_grow", "variance_shrink", "variance_keep", acc / total)


def choose_sensitivity_rank(
    residual_energy: float,
    current_rank: int,
    rank_min: int,
    rank_max: int,
    max_available_rank: int,
    low_threshold: float,
    high_threshold: float,
    step_fraction: float,
) -> RankDecision:
    """Grow when the relative residual energy is above the band, shrink when below it."""
    current = _bounded(current_rank, rank_min, rank_max, max_available_rank)
    lo, hi = sorted((float(low_threshold), float(high_threshold)))
    e = float(residual_energy)
    delta = max(1, int(round(current * max(0.01, float(step_fraction)))))
    if e >= hi:
        target = _bounded(current + delta, rank_min, rank_max, max_available_rank)
        return _decide(target, current, "sensitivity_grow", "sensitivity_grow", "sensitivity_keep_high", e)
    if e <= lo:
        target = _bounded(current - delta, rank_min, rank_max, max_available_rank)
        return _decide(target, current, "sensitivity_shrink", "sensitivity_shrink", "sensitivity_keep_low", e)
    return RankDecision(current, "sensitivity_keep_band", False, e)


def choose_runtime_rank(
    rank_mode: str,
    current_rank: int,
    rank_min: int,
    rank_max: int,
    max_available_rank: int,
    layer_state: Mapping[str, object],
    variance_threshold: float = 0.95,
    sensitivity_low: float = 0.03,
    sensitivity_high: float = 0.10,
    step_fraction: float = 0.125,
) -> RankDecision:
    """Dispatch on ``rank_mode`` in {fixed, variance, sensitivity}."""
    if rank_mode == "fixed":
        target = _bounded(current_rank, rank_min, rank_max, max_available_rank)
        return RankDecision(target, "fixed", target != current_rank, None)
    if rank_mode == "variance":
        return choose_variance_rank(
            layer_state.get("last_coeff_energy_by_rank"), current_rank, rank_min, rank_max, max_available_rank, variance_threshold
        )
    if rank_mode == "sensitivity":
        return choose_sensitivity_rank(
            float(layer_state.get("last_residual_energy", 0.0)), current_rank, rank_min, rank_max, max_available_rank,
            sensitivity_low, sensitivity_high, step_fraction,
        )
    raise ValueError(f"Unsupported rank_mode: {rank_mode}")
