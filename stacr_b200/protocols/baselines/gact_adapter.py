"""Adapter around the optional `gact` activation-quantisation library: enable it when importable, report a skip status otherwise.

Parity: stacr/protocols/baselines/gact_adapter.py of the reference project (status enum, availability and PyTorch
compatibility probes, `try_enable_gact`, a controller object for per-iteration hooks).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ._optional import AdapterResult, AdapterStatus, final_json, probe

GACTStatus = AdapterStatus
GACTResult = AdapterResult
_LEVEL_BITS = {"L0": 32, "L1": 4, "L2": 2, "L3": 2, "L4": 2, "L5": 2}


def check_gact_available() -> Tuple[bool, Optional[str]]:
    ok, info, _ = probe("gact")
    return ok, info


def get_gact_version() -> Optional[str]:
    ok, info, _ = probe("gact")
    return info if ok else None


def check_pytorch_compatibility() -> Tuple[bool, Optional[str]]:
    major = int(torch.__version__.split(".")[0])
    if major >= 2:
        return False, f"gact targets PyTorch 1.x custom autograd internals; running {torch.__version__}"
    return True, None


def _get_bits_for_level(level: str) -> int:
    return _LEVEL_BITS.get(level, 2)


def try_enable_gact(model: nn.Module, level: str = "L2") -> Tuple[nn.Module, AdapterResult]:
    ok, info, mod = probe("gact")
    if not ok:
        return model, AdapterResult(AdapterStatus.SKIPPED_NOT_INSTALLED, str(info))
    if not torch.cuda.is_available():
        return model, AdapterResult(AdapterStatus.SKIPPED_NO_CUDA, "gact kernels need CUDA", info)
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


class GACTController:
    """Owns the (possibly wrapped) model and exposes the per-iteration hook the library expects."""

    def __init__(self, model: nn.Module, level: str = "L2"):
        self.model, self.result = try_enable_gact(model, level)
        self.level = level

    @property
    def enabled(self) -> bool:
        return self.result.ok

    def iterate(self, *args, **kwargs) -> None:
        ctrl = getattr(self.model, "controller", None)
        if self.enabled and ctrl is not None and hasattr(ctrl, "iterate"):
            ctrl.iterate(*args, **kwargs)

    def install_hook(self) -> None:
        ctrl = getattr(self.model, "controller", None)
        if self.enabled and ctrl is not None and hasattr(ctrl, "install_hook"):
            ctrl.install_hook()

    def uninstall_hook(self) -> None:
        ctrl = getattr(self.model, "controller", None)
        if self.enabled and ctrl is not None and hasattr(ctrl, "uninstall_hook"):
            ctrl.uninstall_hook()

    def get_config(self) -> dict:
        return {"baseline": "gact", "level": self.level, "enabled": self.enabled, "bits": _get_bits_for_level(self.level), **self.result.to_dict()}

    def __enter__(self):
        self.install_hook()
        return self

    def __exit__(self, *exc) -> None:
        self.uninstall_hook()


class MockGACTController:
    """Stand-in with the controller's interface that changes nothing, for loops written against the controller."""

    def __init__(self, model: nn.Module, level: str = "L1"):
        self.model, self.level, self.auto_precision, self._iter = model, level, False, 0

    def install_hook(self) -> None:
        return None

    def uninstall_hook(self) -> None:
        return None

    def iterate(self, get_grad_fn=None) -> None:
        self._iter += 1

    @property
    def enabled(self) -> bool:
        return False

    @property
    def iteration(self) -> int:
        return self._iter

    def get_config(self) -> dict:
        return {"baseline": "gact", "level": self.level, "enabled": False, "reason": "mock_controller"}

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        return None


def create_gact_final_json(result: AdapterResult, output_dir: str) -> dict:
    return final_json("gact", result, output_dir)
