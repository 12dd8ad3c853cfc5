"""Byte-driven planners: which layers (or checkpoint boundaries) are worth compressing.

A candidate is kept iff what the dense path would save for backward exceeds what the compressed path stores
(``saved - stored > 0``), unless it is forced or checkpointing already removes the dense save.
Parity: stacr/protocols/planner.py:12-411 of the reference project; ``config`` is any object with the protocol
runner's attribute names (``stacr_rank``, ``stacr_residual_budget``, ``batch_size``, ``max_length`` ...).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Dict, List, Optional, Sequence, Set

import torch
from torch import nn

from ..memory_accounting import bytes_per_elem, stacr_ckpt_stored_bytes, stacr_stored_bytes


@dataclass
class LayerDecision:
    name: str
    keep: bool
    reason: str
    in_features: int
    batch_tokens_est: int
    saved_activation_bytes: int
    stacr_stored_bytes: int
    net_bytes: int
    forced: bool = False

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


@dataclass
class CheckpointSiteDecision:
    name: str
    keep: bool
    reason: str
    hidden_size: int
    batch_tokens_est: int
    saved_boundary_bytes: int
    stacr_stored_bytes: int
    basis_persistent_bytes: int
    net_bytes: int
    forced: bool = False

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


def _module_in_features(module: Optional[nn.Module]) -> Optional[int]:
    if module is None:
        return None
    if isinstance(module, nn.Linear):
        return int(module.in_features)
    if type(module).__name__ == "Conv1D" and hasattr(module, "weight"):
        return int(module.weight.shape[0])
    inner = getattr(module, "in_features", None)
    return int(inner) if inner is not None else None


_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "float16": torch.float16, "fp16": torch.float16,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def _amp_dtype(config: Any) -> torch.dtype:
    amp = str(getattr(getattr(config, "baseline_cfg", None), "amp", getattr(config, "amp", "none"))).lower()
    if amp in ("bf16", "auto"):
        return torch.bfloat16
    return torch.float16 if amp == "fp16" else torch.float32


def _resolve_planner_basis_dtype(config: Any) -> torch.dtype:
    spec = str(getattr(config, "stacr_basis_dtype", "auto")).lower()
    return _DTYPES.get(spec, _amp_dtype(config) if spec in ("auto", "activation") else torch.float32)


def _resolve_planner_saved_tensor_dtype(config: Any) -> torch.dtype:
    return _amp_dtype(config)


def _estimate_batch_tokens(config: Any) -> int:
    return int(getattr(config, "batch_size", 1)) * int(getattr(config, "max_length", getattr(config, "seq_len", 1)))


def _effective_layer_rank(config: Any, *, in_features: int, layer_index: int, total_layers: int) -> int:
    rank = int(getattr(config, "stacr_rank", getattr(config, "rank", 8)))
    if getattr(config, "stacr_adaptive_layer_rank", "none") == "heuristic" and total_layers > 0:
        third = total_layers // 3
        factor = 1.0 if layer_index < third else 0.7 if layer_index < 2 * third else 0.4
        rank = max(min(8, rank), int(rank * factor))
    return max(1, min(rank, in_features))


def _effective_residual_budget(config: Any, *, in_features: int) -> float:
    if str(getattr(config, "stacr_residual_mode", "topk")) == "none":
        return 0.0
    return float(getattr(config, "stacr_residual_budget", getattr(config, "residual_budget", 0.005)))


def _quant_bits(config: Any):
    coeff = 8 if getattr(config, "stacr_quantize_coefficients", False) else None
    res = int(getattr(config, "stacr_residual_quantize_bits", 8)) if getattr(config, "stacr_quantize_residuals", False) else None
    return coeff, res


def _parse_force_names(raw: Optional[str]) -> Set[str]:
    return {p.strip() for p in str(raw).split(",") if p.strip()} if raw else set()


def _checkpointing_eliminates_decoder_mlp_saves(mode: Any) -> bool:
    return str(mode).lower() in ("auto", "transformer_hf", "vision_block", "vision_stage")


def plan_stacr_layers(model: nn.Module, config: Any, candidate_layers: Sequence[str]) -> List[LayerDecision]:
    modules = dict(model.named_modules())
    forced = _parse_force_names(getattr(config, "stacr_force_compress_layers", None))
    stray = sorted(forced - set(candidate_layers))
    if stray:
        raise ValueError("Unknown --stacr-force-compress-layers entries for current candidate set: " + ", ".join(stray))
    tokens = _estimate_batch_tokens(config)
    ckpt = _checkpointing_eliminates_decoder_mlp_saves(getattr(getattr(config, "baseline_cfg", None), "checkpointing", "none"))
    basis_dtype, saved_dtype = _resolve_planner_basis_dtype(config), _resolve_planner_saved_tensor_dtype(config)
    coeff_bits, res_bits = _quant_bits(config)
    floor = int(getattr(config, "stacr_min_features", 0))
    out: List[LayerDecision] = []
    for idx, name in enumerate(candidate_layers):
        width = _module_in_features(modules.get(name))
        skip = "unsupported_module" if width is None else "below_min_features" if floor > 0 and width < floor else None
        if skip:
            if name in forced:
                raise RuntimeError(f"Forced planner keep target '{name}' cannot be compressed ({skip}).")
            out.append(LayerDecision(name, False, skip, -1 if width is None else width, tokens, 0, 0, 0))
            continue
        rank = _effective_layer_rank(config, in_features=width, layer_index=idx, total_layers=len(candidate_layers))
        stored = stacr_stored_bytes(tokens, width, rank, _effective_residual_budget(config, in_features=width), saved_dtype,
                                    coeff_bits=coeff_bits, residual_bits=res_bits, basis_dtype=basis_dtype, include_meta=False).total_bytes
        saved = 0 if ckpt else tokens * width * bytes_per_elem(saved_dtype)
        net = saved - stored
        if name in forced:
            keep, why = True, "forced_keep"
        elif ckpt:
            keep, why = False, "checkpointing_zero_save"
        else:
            keep, why = (True, "positive_net") if net > 0 else (False, "non_positive_net")
        out.append(LayerDecision(name, keep, why, width, tokens, saved, stored, net, name in forced))
    return out


def summarize_layer_decisions(decisions: Sequence[LayerDecision]) -> Dict[str, Any]:
    kept = [d for d in decisions if d.keep]
    reasons: Dict[str, int] = {}
    for d in decisions:
        reasons[d.reason] = reasons.get(d.reason, 0) + 1
    return {"candidates": len(decisions), "kept": len(kept), "kept_names": [d.name for d in kept], "reasons": reasons,
            "net_bytes_kept": sum(d.net_bytes for d in kept), "stored_bytes_kept": sum(d.stacr_stored_bytes for d in kept)}


def plan_stacr_checkpoint_sites(model: nn.Module, config: Any, sites: Sequence[str], hidden_size: int) -> List[CheckpointSiteDecision]:
    """Same rule for checkpoint boundaries: dense boundary ``tokens x hidden`` vs int8 coefficients + per-row scales + basis."""
    forced = _parse_force_names(getattr(config, "stacr_force_checkpoint_sites", None))
    tokens = _estimate_batch_tokens(config)
    dtype = _resolve_planner_saved_tensor_dtype(config)
    rank = max(1, min(int(getattr(config, "stacr_checkpoint_rank", getattr(config, "stacr_rank", 32))), hidden_size))
    basis = hidden_size * rank * 4
    out = []
    for name in sites:
        saved = tokens * hidden_size * bytes_per_elem(dtype)
        stored = stacr_ckpt_stored_bytes(tokens, hidden_size, rank, dtype)
        net = saved - stored - basis
        if name in forced:
            keep, why = True, "forced_keep"
        else:
            keep, why = (True, "positive_net") if net > 0 else (False, "non_positive_net")
        out.append(CheckpointSiteDecision(name, keep, why, hidden_size, tokens, saved, stored, basis, net, name in forced))
    return out


def summarize_checkpoint_site_decisions(decisions: Sequence[CheckpointSiteDecision]) -> Dict[str, Any]:
    kept = [d for d in decisions if d.keep]
    return {"sites": len(decisions), "kept": len(kept), "kept_names": [d.name for d in kept], "net_bytes_kept": sum(d.net_bytes for d in kept)}
