"""Adapter around the optional `actnn` activation-quantisation library: enable it when importable, report a skip status otherwise.

Parity: stacr/protocols/baselines/actnn_adapter.py of the reference project (status enum, availability and PyTorch
compatibility probes, `try_enable_actnn`, a controller object for per-iteration hooks).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ._optional import AdapterResult, AdapterStatus, final_json, probe

ACTNNStatus = AdapterStatus
ACTNNResult = AdapterResult
ActNNStatus = AdapterStatus
ActNNResult = AdapterResult
_LEVEL_BITS = {"L0": 32, "L1": 4, "L2": 2, "L3": 2, "L4": 2, "L5": 2}


def check_actnn_available() -> Tuple[bool, Optional[str]]:
    ok, info, _ = probe("actnn")
    return ok, info


def get_actnn_version() -> Optional[str]:
    ok, info, _ = probe("actnn")
    return info if ok else None


def check_pytorch_compatibility() -> Tuple[bool, Optional[str]]:
    major = int(torch.__version__.split(".")[0])
    if major >= 2:
        return False, f"actnn targets PyTorch 1.x custom autograd internals; running {torch.__version__}"
    return True, None


def _get_bits_for_level(level: str) -> int:
    return _LEVEL_BITS.get(level, 2)


def try_enable_actnn(model: nn.Module, level: str = "L2") -> Tuple[nn.Module, AdapterResult]:
    ok, info, mod = probe("actnn")
    if not ok:
        return model, AdapterResult(AdapterStatus.SKIPPED_NOT_INSTALLED, str(info))
    if not torch.cuda.is_available():
        return model, AdapterResult(AdapterStatus.SKIPPED_NO_CUDA, "actnn kernels need CUDA", info)
    compatible, why = check_pytorch_compatibility()
    if not compatible:
        return model, AdapterResult(AdapterStatus.SKIPPED_INCOMPATIBLE, why or "", info)
    try:
        if hasattr(mod, "set_optimization_level"):
            mod.set_optimization_level(level)
        converter = getattr(mod, "QModule", None)
        wrapped = converter(model) if converter is not None else model
        return wrapped, AdapterResult(AdapterStatus.OK, version=info, details={"level": level, "bits": _get_bits_for_level(level)})
    except Exception as exc:  # noqa: BLE001
        return model, AdapterResult(AdapterStatus.ERROR, f"{type(exc).__name__}: {exc}", info)


class ACTNNController:
    """Owns the (possibly wrapped) model and exposes the per-iteration hook the library expects."""

    def __init__(self, model: nn.Module, level: str = "L2"):
        self.model, self.result = try_enable_actnn(model, level)
        self.level = level

    @property
    def enabled(self) -> bool:
        return self.result.ok

    def iterate(self, *args, **kwargs) -> None:
        ctrl = getattr(self.model, "controller", None)
        if self.enabled and ctrl is not None and hasattr(ctrl, "iterate"):
            ctrl.iterate(*args, **kwargs)

    def get_config(self) -> dict:
        return {"baseline": "actnn", "level": self.level, "enabled": self.enabled, "bits": _get_bits_for_level(self.level), **self.result.to_dict()}

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        return None


ActNNController = ACTNNController


def create_actnn_final_json(result: AdapterResult, output_dir: str) -> dict:
    return final_json("actnn", result, output_dir)
