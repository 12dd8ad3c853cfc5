"""Mixed-precision baseline (parity: stacr/protocols/baselines/amp.py:16-168 of the reference project)."""

from __future__ import annotations

from contextlib import nullcontext
from typing import Optional, Tuple

import torch


def _is_bf16_supported(device: str) -> bool:
    if not str(device).startswith("cuda"):
        return True
    return torch.cuda.is_available() and torch.cuda.is_bf16_supported()


def resolve_amp_dtype(amp_mode: str, device: str = "cuda") -> Tuple[Optional[torch.dtype], bool]:
    """``(autocast dtype or None, needs GradScaler)`` for ``none | auto | bf16 | fp16``."""
    mode = str(amp_mode).lower()
    if mode in ("none", "off", "false", "fp32"):
        return None, False
    on_cuda = str(device).startswith("cuda")
    if mode == "auto":
        if _is_bf16_supported(device):
            return torch.bfloat16, False
        return (torch.float16, True) if on_cuda else (None, False)
    if mode in ("bf16", "bfloat16"):
        if not _is_bf16_supported(device):
            raise ValueError("bf16 autocast requested but the device does not support it")
        return torch.bfloat16, False
    if mode in ("fp16", "float16"):
        if not on_cuda:
            raise ValueError("fp16 autocast requires CUDA")
        return torch.float16, True
    raise ValueError(f"Unknown amp mode: {amp_mode!r}")


def amp_context(amp_mode: str, device: str = "cuda"):
    dtype, _ = resolve_amp_dtype(amp_mode, device)
    if dtype is None:
        return nullcontext()
    return torch.autocast(device_type="cuda" if str(device).startswith("cuda") else "cpu", dtype=dtype)


class AMPManager:
    """Autocast + (for fp16) loss scaling behind one object: ``autocast()``, ``backward(loss)``, ``step(optimizer)``."""

    def __init__(self, amp_mode: str, device: str = "cuda"):
        self.amp_mode, self.device = amp_mode, str(device)
        self.dtype, needs_scaler = resolve_amp_dtype(amp_mode, device)
        self.scaler = torch.amp.GradScaler("cuda", enabled=True) if needs_scaler else None

    @property
    def enabled(self) -> bool:
        return self.dtype is not None

    def autocast(self):
        if not self.enabled:
            return nullcontext()
        return torch.autocast(device_type="cuda" if self.device.startswith("cuda") else "cpu", dtype=self.dtype)

    def backward(self, loss: torch.Tensor) -> None:
        (self.scaler.scale(loss) if self.scaler else loss).backward()

    def unscale_(self, optimizer) -> None:
        if self.scaler:
            self.scaler.unscale_(optimizer)

    def step(self, optimizer: torch.optim.Optimizer) -> None:
        if self.scaler:
            self.scaler.step(optimizer)
            self.scaler.update()
        else:
            optimizer.step()

    def get_scale(self) -> float:
        return float(self.scaler.get_scale()) if self.scaler else 1.0

    def state_dict(self) -> dict:
        return {"amp_mode": self.amp_mode, "scaler": self.scaler.state_dict() if self.scaler else None}

    def load_state_dict(self, state_dict: dict) -> None:
        if self.scaler and state_dict.get("scaler"):
            self.scaler.load_state_dict(state_dict["scaler"])
