"""GaLore as a protocol baseline: availability probes, a configuration record and an optimizer factory with a status.

The optimizer itself lives with the comparators (``stacr_b200.comparators.lowrank_optim.GaLoreAdamW``, or the
``galore_torch`` package when installed and preferred); this module adds the status-reporting surface the
protocol runner and sweeps use.  Parity: stacr/protocols/baselines/galore_adapter.py:14-260.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from ...comparators.galore_adapter import create_galore_optimizer as _build, galore_available  # noqa: F401
from ._optional import AdapterResult, AdapterStatus, final_json, probe

GaLoreStatus = AdapterStatus
GaLoreResult = AdapterResult

__all__ = ["GaLoreStatus", "GaLoreResult", "GaLoreConfig", "check_galore_available", "check_pytorch_version", "get_galore_version",
           "create_galore_optimizer", "try_enable_galore", "parse_galore_config_string", "create_galore_final_json", "galore_available"]


@dataclass
class GaLoreConfig:
    rank: int = 128
    update_proj_gap: int = 200
    scale: float = 0.25
    proj_type: str = "std"


def check_galore_available() -> Tuple[bool, Optional[str]]:
    """Always available: the in-tree optimizer serves when ``galore_torch`` is not installed (the note says which)."""
    ok, info, _ = probe("galore_torch")
    return True, (f"galore_torch {info}" if ok else "in-tree GaLoreAdamW")


def check_pytorch_version() -> Tuple[bool, Optional[str]]:
    major = int(torch.__version__.split(".")[0])
    return (True, None) if major >= 2 else (False, f"GaLore needs PyTorch >= 2.0, running {torch.__version__}")


def get_galore_version() -> Optional[str]:
    ok, info, _ = probe("galore_torch")
    return info if ok else "in-tree"


def create_galore_optimizer(model, lr: float = 0.01, weight_decay: float = 0.0, config: Optional[GaLoreConfig] = None,
                            target_modules: Optional[List[str]] = None, prefer_external: bool = False):
    """``(optimizer or None, result)``; the low-rank groups are the 2-D weights of modules matching ``target_modules``."""
    cfg = config or GaLoreConfig()
    compatible, why = check_pytorch_version()
    if not compatible:
        return None, AdapterResult(AdapterStatus.SKIPPED_INCOMPATIBLE, why or "")
    try:
        opt = _build(model, lr=lr, rank=cfg.rank, update_proj_gap=cfg.update_proj_gap, scale=cfg.scale, proj_type=cfg.proj_type,
                     weight_decay=weight_decay, target_modules=target_modules, prefer_external=prefer_external)
    except Exception as exc:  # noqa: BLE001
        return None, AdapterResult(AdapterStatus.ERROR, f"{type(exc).__name__}: {exc}")
    low = sum(len(g["params"]) for g in opt.param_groups if "rank" in g)
    return opt, AdapterResult(AdapterStatus.OK, "GaLore enabled", get_galore_version(),
                              {"rank": cfg.rank, "update_proj_gap": cfg.update_proj_gap, "scale": cfg.scale, "proj_type": cfg.proj_type,
                               "low_rank_params": low, "implementation": type(opt).__module__})


def try_enable_galore(model, lr: float = 0.01, weight_decay: float = 0.0, rank: int = 128, update_proj_gap: int = 200, scale: float = 0.25,
                      proj_type: str = "std", target_modules: Optional[List[str]] = None):
    return create_galore_optimizer(model, lr, weight_decay, GaLoreConfig(rank, update_proj_gap, scale, proj_type), target_modules)


def parse_galore_config_string(text: str) -> Optional[GaLoreConfig]:
    """``"rank=128,update_gap=200,scale=0.25,type=std"`` as a configuration; ``None`` for empty, ``"none"`` or unparsable text."""
    if not text or text.strip().lower() == "none":
        return None
    cfg = GaLoreConfig()
    casts = {"rank": ("rank", int), "update_gap": ("update_proj_gap", int), "update_proj_gap": ("update_proj_gap", int),
             "scale": ("scale", float), "proj_type": ("proj_type", str), "type": ("proj_type", str)}
    try:
        for item in text.split(","):
            key, sep, value = item.partition("=")
            if sep and key.strip().lower() in casts:
                name, cast = casts[key.strip().lower()]
                setattr(cfg, name, cast(value.strip()))
    except ValueError:
        return None
    return cfg


def create_galore_final_json(result: AdapterResult, output_dir: str) -> dict:
    return final_json("galore", result, output_dir)
