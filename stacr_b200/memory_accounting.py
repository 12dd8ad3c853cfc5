"""Stored-bytes calculators and budget planners for SVD, tensor-train, Tucker and STAC-R factors.

Each method has three pieces: ``*_stored_elements`` / ``*_stored_bytes`` (what one saved activation
costs), ``*_rank_from_budget`` (largest rank that fits a byte budget) and ``plan_*`` (a ``PlanResult``
with feasibility, reason code, achieved ratio and a storage breakdown).  API parity:
stacr/memory_accounting.py:37-1882 of the reference project.
"""

from __future__ import annotations

import math
import sys
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

META_INT_BYTES = 4


class FeasibilityReason(Enum):
    FEASIBLE = "feasible"
    BUDGET_TOO_LOW_FOR_MIN_PARAMS = "budget_too_low_for_min_params"
    TARGET_RATIO_EXCEEDS_RHO_MAX = "target_ratio_exceeds_rho_max"
    INVALID_PARAMETERS = "invalid_parameters"
    EXCEEDS_METHOD_MAX_RANK = "exceeds_method_max_rank"
    UNSUPPORTED_SHAPE = "unsupported_shape"


class SigmaStorage(Enum):
    VECTOR = "vector"  # k singular values
    MATRIX = "matrix"  # k x k
    FOLDED = "folded"  # folded into U


@dataclass
class StorageBreakdown:
    total_bytes: int
    payload_bytes: int
    meta_bytes: int
    persistent_cache_bytes: int = 0
    details: Dict[str, Any] = field(default_factory=dict)

    def __repr__(self):
        return f"StorageBreakdown(total={self.total_bytes}, payload={self.payload_bytes}, meta={self.meta_bytes})"


@dataclass
class PlanResult:
    feasible: bool
    reason: FeasibilityReason
    original_bytes: int
    budget_bytes: Optional[int] = None
    stored_bytes: Optional[int] = None
    achieved_ratio: Optional[float] = None
    k: Optional[int] = None
    ranks: Optional[List[int]] = None
    rho_max: Optional[float] = None
    breakdown: Optional[StorageBreakdown] = None
    shape: Optional[Tuple[int, ...]] = None
    method: Optional[str] = None

    def to_dict(self) -> Dict[str, Any]:
        b = self.breakdown
        return {
            "feasible": self.feasible, "reason": self.reason.value, "original_bytes": self.original_bytes,
            "budget_bytes": self.budget_bytes, "stored_bytes": self.stored_bytes, "achieved_ratio": self.achieved_ratio,
            "k": self.k, "ranks": self.ranks, "rho_max": self.rho_max, "shape": list(self.shape) if self.shape else None,
            "method": self.method,
            "breakdown": None if b is None else {"total_bytes": b.total_bytes, "payload_bytes": b.payload_bytes,
                                                 "meta_bytes": b.meta_bytes, "details": b.details},
        }


# ------------------------------------------------------------------------------ basics
def bytes_per_elem(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def original_bytes(shape: Tuple[int, ...], dtype: torch.dtype) -> int:
    return math.prod(int(d) for d in shape) * bytes_per_elem(dtype)


def original_bytes_from_tensor(tensor: torch.Tensor) -> int:
    return tensor.numel() * tensor.element_size()


def meta_bytes(shape_len: int, perm_len: int = 0, ranks_len: int = 0, extra_fields: int = 2, meta_int_bytes: int = META_INT_BYTES) -> int:
    """Bookkeeping ints stored with a packed tensor: shape, permutation, ranks, method id + flags."""
    return (shape_len + perm_len + ranks_len + extra_fields) * meta_int_bytes


def _breakdown(payload: int, meta: int, details: dict, persistent: int = 0) -> StorageBreakdown:
    return StorageBreakdown(payload + meta, payload, meta, persistent, details)


def _resolve_budget(orig: int, budget_bytes, target_ratio):
    if (budget_bytes is None) == (target_ratio is None):
        raise ValueError("Specify exactly one of budget_bytes or target_ratio")
    if target_ratio is not None:
        if target_ratio <= 0:
            raise ValueError("target_ratio must be positive")
        return int(orig / target_ratio)
    return int(budget_bytes)


def _finish(method, shape, orig, budget, stored_fn, rank_or_ranks, rho_max, target_ratio) -> PlanResult:
    """Common tail of the planners: build the result for the chosen rank(s) or explain infeasibility."""
    if rank_or_ranks is None:
        reason = FeasibilityReason.TARGET_RATIO_EXCEEDS_RHO_MAX if target_ratio is not None else FeasibilityReason.BUDGET_TOO_LOW_FOR_MIN_PARAMS
        return PlanResult(False, reason, orig, budget, rho_max=rho_max, shape=tuple(shape), method=method)
    bd = stored_fn(rank_or_ranks)
    is_list = isinstance(rank_or_ranks, (list, tuple))
    return PlanResult(True, FeasibilityReason.FEASIBLE, orig, budget, bd.total_bytes, orig / bd.total_bytes if bd.total_bytes else None,
                      k=None if is_list else int(rank_or_ranks), ranks=list(rank_or_ranks) if is_list else None, rho_max=rho_max,
                      breakdown=bd, shape=tuple(shape), method=method)


# ------------------------------------------------------------------------------ SVD
def svd_stored_elements(batch: int, features: int, rank: int, store_sigma: SigmaStorage = SigmaStorage.VECTOR) -> int:
    sigma = {SigmaStorage.VECTOR: rank, SigmaStorage.MATRIX: rank * rank, SigmaStorage.FOLDED: 0}[store_sigma]
    return batch * rank + rank * features + sigma


def svd_stored_bytes(batch, features, rank, dtype, store_sigma=SigmaStorage.VECTOR, include_meta=True) -> StorageBreakdown:
    payload = svd_stored_elements(batch, features, rank, store_sigma) * bytes_per_elem(dtype)
    meta = meta_bytes(2, ranks_len=1) if include_meta else 0
    return _breakdown(payload, meta, {"rank": rank, "sigma": store_sigma.value})


def svd_rho_max(batch, features, dtype, store_sigma=SigmaStorage.VECTOR, include_meta=True) -> float:
    """Best achievable compression ratio (rank 1)."""
    return original_bytes((batch, features), dtype) / svd_stored_bytes(batch, features, 1, dtype, store_sigma, include_meta).total_bytes


def svd_rank_from_budget(batch, features, dtype, budget_bytes, store_sigma=SigmaStorage.VECTOR, include_meta=True) -> Optional[int]:
    best = None
    for k in range(1, min(batch, features) + 1):
        if svd_stored_bytes(batch, features, k, dtype, store_sigma, include_meta).total_bytes > budget_bytes:
            break
        best = k
    return best


def svd_rank_from_ratio(batch, features, dtype, target_ratio, store_sigma=SigmaStorage.VECTOR, include_meta=True) -> Optional[int]:
    return svd_rank_from_budget(batch, features, dtype, int(original_bytes((batch, features), dtype) / target_ratio), store_sigma, include_meta)


def plan_svd(batch, features, dtype, budget_bytes=None, target_ratio=None, store_sigma=SigmaStorage.VECTOR, include_meta=True) -> PlanResult:
    orig = original_bytes((batch, features), dtype)
    if batch < 1 or features < 1:
        return PlanResult(False, FeasibilityReason.INVALID_PARAMETERS, orig, shape=(batch, features), method="svd")
    budget = _resolve_budget(orig, budget_bytes, target_ratio)
    k = svd_rank_from_budget(batch, features, dtype, budget, store_sigma, include_meta)
    return _finish("svd", (batch, features), orig, budget, lambda r: svd_stored_bytes(batch, features, r, dtype, store_sigma, include_meta),
                   k, svd_rho_max(batch, features, dtype, store_sigma, include_meta), target_ratio)


# ------------------------------------------------------------------------------ tensor train
def tt_stored_elements(dims: Sequence[int], tt_ranks: Sequence[int]) -> int:
    """Cores ``G_i`` of shape ``r_{i-1} x d_i x r_i`` with ``r_0 = r_d = 1`` (``tt_ranks`` has ``len(dims)+1`` entries)."""
    if len(tt_ranks) != len(dims) + 1:
        raise ValueError("tt_ranks must have len(dims)+1 entries")
    return sum(int(tt_ranks[i]) * int(d) * int(tt_ranks[i + 1]) for i, d in enumerate(dims))


def tt_uniform_ranks(dims: Sequence[int], rank: int) -> List[int]:
    """Uniform internal rank clipped by what the unfoldings allow."""
    n = len(dims)
    out = [1]
    for i in range(1, n):
        left, right = math.prod(dims[:i]), math.prod(dims[i:])
        out.append(max(1, min(int(rank), left, right)))
    return out + [1]


def tt_stored_bytes(dims, tt_ranks, dtype, include_meta=True) -> StorageBreakdown:
    payload = tt_stored_elements(dims, tt_ranks) * bytes_per_elem(dtype)
    meta = meta_bytes(len(dims), ranks_len=len(tt_ranks)) if include_meta else 0
    return _breakdown(payload, meta, {"tt_ranks": list(tt_ranks)})


def tt_rank_from_budget(dims, dtype, budget_bytes, include_meta=True, max_rank: Optional[int] = None) -> Optional[List[int]]:
    limit = max_rank or max(1, max(min(math.prod(dims[:i]), math.prod(dims[i:])) for i in range(1, len(dims))) if len(dims) > 1 else 1)
    best = None
    for r in range(1, limit + 1):
        ranks = tt_uniform_ranks(dims, r)
        if tt_stored_bytes(dims, ranks, dtype, include_meta).total_bytes > budget_bytes:
            break
        best = ranks
    return best


def plan_tt(shape, dtype, budget_bytes=None, target_ratio=None, include_meta=True) -> PlanResult:
    dims = [int(d) for d in shape]
    orig = original_bytes(tuple(dims), dtype)
    if len(dims) < 2:
        return PlanResult(False, FeasibilityReason.UNSUPPORTED_SHAPE, orig, shape=tuple(dims), method="tt")
    budget = _resolve_budget(orig, budget_bytes, target_ratio)
    ranks = tt_rank_from_budget(dims, dtype, budget, include_meta)
    rho = orig / tt_stored_bytes(dims, tt_uniform_ranks(dims, 1), dtype, include_meta).total_bytes
    return _finish("tt", dims, orig, budget, lambda rk: tt_stored_bytes(dims, rk, dtype, include_meta), ranks, rho, target_ratio)


def validate_tt_ranks(dims: Sequence[int], tt_ranks: Sequence[int]) -> Tuple[bool, str]:
    if len(tt_ranks) != len(dims) + 1:
        return False, "tt_ranks must have len(dims)+1 entries"
    if tt_ranks[0] != 1 or tt_ranks[-1] != 1:
        return False, "boundary TT ranks must be 1"
    for i in range(1, len(dims)):
        if tt_ranks[i] < 1 or tt_ranks[i] > min(math.prod(dims[:i]), math.prod(dims[i:])):
            return False, f"rank {i} out of range"
    return True, "ok"


# ------------------------------------------------------------------------------ Tucker
def tucker_stored_elements(dims: Sequence[int], ranks: Sequence[int]) -> int:
    if len(dims) != len(ranks):
        raise ValueError("ranks must match dims")
    return math.prod(int(r) for r in ranks) + sum(int(d) * int(r) for d, r in zip(dims, ranks))


def tucker_uniform_ranks(dims: Sequence[int], rank: int) -> List[int]:
    return [max(1, min(int(rank), int(d))) for d in dims]


def tucker_proportional_ranks(dims: Sequence[int], alpha: float, min_rank: int = 1) -> List[int]:
    return [max(int(min_rank), min(int(d), int(round(alpha * d)))) for d in dims]


def tucker_stored_bytes(dims, ranks, dtype, include_meta=True) -> StorageBreakdown:
    payload = tucker_stored_elements(dims, ranks) * bytes_per_elem(dtype)
    meta = meta_bytes(len(dims), ranks_len=len(ranks)) if include_meta else 0
    return _breakdown(payload, meta, {"ranks": list(ranks)})


def tucker_rank_from_budget(dims, dtype, budget_bytes, include_meta=True) -> Optional[List[int]]:
    best = None
    for r in range(1, max(dims) + 1):
        ranks = tucker_uniform_ranks(dims, r)
        if tucker_stored_bytes(dims, ranks, dtype, include_meta).total_bytes > budget_bytes:
            break
        best = ranks
    return best


def tucker_proportional_ranks_from_budget(dims, dtype, budget_bytes, include_meta=True, steps: int = 200) -> Optional[List[int]]:
    best = None
    for i in range(1, steps + 1):
        ranks = tucker_proportional_ranks(dims, i / steps)
        if tucker_stored_bytes(dims, ranks, dtype, include_meta).total_bytes > budget_bytes:
            break
        best = ranks
    return best


def plan_tucker(shape, dtype, budget_bytes=None, target_ratio=None, include_meta=True, proportional: bool = False) -> PlanResult:
    dims = [int(d) for d in shape]
    orig = original_bytes(tuple(dims), dtype)
    if len(dims) < 2:
        return PlanResult(False, FeasibilityReason.UNSUPPORTED_SHAPE, orig, shape=tuple(dims), method="tucker")
    budget = _resolve_budget(orig, budget_bytes, target_ratio)
    pick = tucker_proportional_ranks_from_budget if proportional else tucker_rank_from_budget
    ranks = pick(dims, dtype, budget, include_meta)
    rho = orig / tucker_stored_bytes(dims, [1] * len(dims), dtype, include_meta).total_bytes
    return _finish("tucker", dims, orig, budget, lambda rk: tucker_stored_bytes(dims, rk, dtype, include_meta), ranks, rho, target_ratio)


def validate_tucker_ranks(dims: Sequence[int], ranks: Sequence[int]) -> Tuple[bool, str]:
    if len(dims) != len(ranks):
        return False, "ranks must match dims"
    for d, r in zip(dims, ranks):
        if r < 1 or r > d:
            return False, f"rank {r} out of range for dim {d}"
    return True, "ok"


# ------------------------------------------------------------------------------ STAC-R
def stacr_stored_elements(batch: int, features: int, rank: int, residual_budget: float = 0.0) -> int:
    """Coefficients ``batch x rank`` plus ``floor(budget * batch * features)`` residual entries (the basis is persistent)."""
    return batch * rank + int(batch * features * residual_budget)


def stacr_stored_bytes(batch, features, rank, residual_budget=0.0, dtype=torch.float32, coeff_bits=None, residual_bits=None,
                       basis_dtype=None, include_meta=True, include_basis=False) -> StorageBreakdown:
    vb = bytes_per_elem(dtype)
    pack = lambda count, bits: math.ceil(count * bits / 8) if bits else count * vb
    n_coeff, n_res = batch * rank, int(batch * features * residual_budget)
    coeff = pack(n_coeff, coeff_bits) + (vb if coeff_bits and n_coeff else 0)
    total_cells = batch * features
    idx_b = 2 if total_cells < 32768 else 4 if total_cells <= 2**31 else 8
    res_vals = pack(n_res, residual_bits) + (vb if residual_bits and n_res else 0)
    basis = features * rank * bytes_per_elem(basis_dtype or dtype)
    payload = coeff + res_vals + n_res * idx_b + (basis if include_basis else 0)
    meta = meta_bytes(2, ranks_len=1, extra_fields=4) if include_meta else 0
    return _breakdown(payload, meta, {"coeff_bytes": coeff, "residual_value_bytes": res_vals, "residual_index_bytes": n_res * idx_b,
                                      "basis_bytes": basis, "rank": rank, "residual_count": n_res}, persistent=0 if include_basis else basis)


def stacr_ckpt_stored_bytes(batch, features, rank, dtype=torch.float32, coeff_bits: Optional[int] = 8, per_row_scale: bool = True) -> int:
    """Checkpoint-boundary codec: int8 coefficients with one scale per row, basis persistent."""
    vb = bytes_per_elem(dtype)
    coeff = math.ceil(batch * rank * coeff_bits / 8) if coeff_bits else batch * rank * vb
    return coeff + (batch * 4 if per_row_scale and coeff_bits else 0)


def stacr_rho_max(batch, features, dtype, residual_budget=0.0, coeff_bits=None, residual_bits=None, include_meta=True) -> float:
    return original_bytes((batch, features), dtype) / stacr_stored_bytes(batch, features, 1, residual_budget, dtype, coeff_bits, residual_bits,
                                                                         include_meta=include_meta).total_bytes


def stacr_rank_from_budget(batch, features, dtype, budget_bytes, residual_budget=0.0, coeff_bits=None, residual_bits=None,
                           basis_dtype=None, include_meta=True) -> Optional[int]:
    best = None
    for r in range(1, features + 1):
        if stacr_stored_bytes(batch, features, r, residual_budget, dtype, coeff_bits, residual_bits, basis_dtype, include_meta).total_bytes > budget_bytes:
            break
        best = r
    return best


def plan_stacr(batch, features, dtype, budget_bytes=None, target_ratio=None, residual_budget=0.1, coeff_bits=None, residual_bits=None,
               basis_dtype=None, include_meta=True) -> PlanResult:
    orig = original_bytes((batch, features), dtype)
    if batch < 1 or features < 1 or not 0 <= residual_budget <= 1:
        return PlanResult(False, FeasibilityReason.INVALID_PARAMETERS, orig, shape=(batch, features), method="stacr")
    budget = _resolve_budget(orig, budget_bytes, target_ratio)
    k = stacr_rank_from_budget(batch, features, dtype, budget, residual_budget, coeff_bits, residual_bits, basis_dtype, include_meta)
    stored = lambda r: stacr_stored_bytes(batch, features, r, residual_budget, dtype, coeff_bits, residual_bits, basis_dtype, include_meta)
    return _finish("stacr", (batch, features), orig, budget, stored, k,
                   stacr_rho_max(batch, features, dtype, residual_budget, coeff_bits, residual_bits, include_meta), target_ratio)


# ------------------------------------------------------------------------------ comparisons / reporting
def _tensorize(n: int) -> List[int]:
    """Split ``n`` into two near-square factors (for applying TT/Tucker to matrices)."""
    a = int(math.isqrt(n))
    while a > 1 and n % a:
        a -= 1
    return [a, n // a] if a > 1 else [n]


def compare_methods_at_budget(shape, dtype, budget_bytes, include_meta=True) -> Dict[str, PlanResult]:
    shape = tuple(int(d) for d in shape)
    out: Dict[str, PlanResult] = {}
    if len(shape) == 2:
        out["svd"] = plan_svd(shape[0], shape[1], dtype, budget_bytes=budget_bytes, include_meta=include_meta)
        out["stacr"] = plan_stacr(shape[0], shape[1], dtype, budget_bytes=budget_bytes, residual_budget=0.005, include_meta=include_meta)
        dims = _tensorize(shape[0]) + _tensorize(shape[1])
    else:
        dims = list(shape)
    out["tt"] = plan_tt(dims, dtype, budget_bytes=budget_bytes, include_meta=include_meta)
    out["tucker"] = plan_tucker(dims, dtype, budget_bytes=budget_bytes, include_meta=include_meta)
    return out


def format_plan_result(result: PlanResult) -> str:
    if not result.feasible:
        return f"[{result.method}] infeasible: {result.reason.value} (original {result.original_bytes} B, budget {result.budget_bytes} B)"
    what = f"k={result.k}" if result.k is not None else f"ranks={result.ranks}"
    return f"[{result.method}] {what} stored {result.stored_bytes} B of {result.original_bytes} B (ratio {result.achieved_ratio:.2f}x, rho_max {result.rho_max:.1f}x)"


@dataclass
class LayerMemoryPlan:
    layer_name: str
    shape: Tuple[int, ...]
    original_bytes: int
    budget_bytes: int
    method: str
    plan_result: PlanResult


def print_memory_table(layer_plans: List[LayerMemoryPlan], file=None) -> str:
    lines = [f"{'layer':40s} {'shape':>18s} {'orig MB':>9s} {'budget MB':>10s} {'method':>7s} {'stored MB':>10s} {'ratio':>7s} status"]
    tot_o = tot_s = 0
    for lp in layer_plans:
        r = lp.plan_result
        stored = r.stored_bytes or 0
        tot_o += lp.original_bytes
        tot_s += stored if r.feasible else lp.original_bytes
        lines.append(f"{lp.layer_name[:40]:40s} {str(tuple(lp.shape)):>18s} {lp.original_bytes / 1e6:9.2f} {lp.budget_bytes / 1e6:10.2f} "
                     f"{lp.method:>7s} {stored / 1e6:10.2f} {(r.achieved_ratio or 0):7.2f} {r.reason.value}")
    lines.append(f"{'TOTAL':40s} {'':>18s} {tot_o / 1e6:9.2f} {'':>10s} {'':>7s} {tot_s / 1e6:10.2f} {(tot_o / tot_s if tot_s else 0):7.2f}")
    text = "\n".join(lines)
    print(text, file=file or sys.stdout)
    return text


def plan_layers_for_debug(named_shapes, dtype, ratio: float, method: str = "stacr", **kw) -> List[LayerMemoryPlan]:
    """Plan every ``(name, shape)`` at a common compression ratio."""
    plans = []
    for name, shape in named_shapes:
        shape = tuple(int(d) for d in shape)
        orig = original_bytes(shape, dtype)
        budget = int(orig / ratio)
        if method == "svd":
            res = plan_svd(shape[0], shape[1], dtype, budget_bytes=budget)
        elif method == "tt":
            res = plan_tt(shape, dtype, budget_bytes=budget)
        elif method == "tucker":
            res = plan_tucker(shape, dtype, budget_bytes=budget)
        else:
            res = plan_stacr(math.prod(shape[:-1]), shape[-1], dtype, budget_bytes=budget, **kw)
        plans.append(LayerMemoryPlan(name, shape, orig, budget, method, res))
    return plans


def debug_memory_accounting(model, rows: int, dtype=torch.float16, ratio: float = 4.0, method: str = "stacr", file=None) -> str:
    """Print the plan table for every linear layer of ``model`` seeing ``rows`` activation rows."""
    shapes = [(n, (rows, m.in_features)) for n, m in model.named_modules() if hasattr(m, "in_features")]
    return print_memory_table(plan_layers_for_debug(shapes, dtype, ratio, method), file=file)
