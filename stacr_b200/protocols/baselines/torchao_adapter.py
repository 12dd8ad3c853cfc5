"""Adapter around optional ``torchao`` low-bit optimizers / float8 training (graceful skip when absent).

Parity: stacr/protocols/baselines/torchao_adapter.py of the reference project.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._optional import AdapterResult, AdapterStatus, probe

TorchAOStatus = AdapterStatus
TorchAOResult = AdapterResult


def check_torchao_available() -> Tuple[bool, Optional[str]]:
    ok, info, _ = probe("torchao")
    return ok, info


def try_create_torchao_optimizer(params, name: str = "adamw8bit", lr: float = 5e-5, weight_decay: float = 0.01, **kw):
    ok, info, _ = probe("torchao")
    if not ok:
        return None, AdapterResult(AdapterStatus.SKIPPED_NOT_INSTALLED, str(info))
    found, err, mod = probe("torchao.optim")
    if not found:
        found, err, mod = probe("torchao.prototype.low_bit_optim")
    if not found:
        return None, AdapterResult(AdapterStatus.SKIPPED_INCOMPATIBLE, str(err), info)
    table = {"adamw8bit": "AdamW8bit", "adamw4bit": "AdamW4bit", "adamwfp8": "AdamWFp8"}
    cls = getattr(mod, table.get(name.lower(), ""), None)
    if cls is None:
        return None, AdapterResult(AdapterStatus.SKIPPED_INCOMPATIBLE, f"torchao has no optimizer {name!r}", info)
    try:
        return cls(params, lr=lr, weight_decay=weight_decay, **kw), AdapterResult(AdapterStatus.OK, version=info, details={"optimizer": name})
    except Exception as exc:  # noqa: BLE001
        return None, AdapterResult(AdapterStatus.ERROR, f"{type(exc).__name__}: {exc}", info)


def try_enable_float8_training(model: torch.nn.Module):
    ok, info, _ = probe("torchao")
    if not ok:
        return model, AdapterResult(AdapterStatus.SKIPPED_NOT_INSTALLED, str(info))
    found, err, mod = probe("torchao.float8")
    if not found or not hasattr(mod, "convert_to_float8_training"):
        return model, AdapterResult(AdapterStatus.SKIPPED_INCOMPATIBLE, str(err), info)
    if not torch.cuda.is_available():
        return model, AdapterResult(AdapterStatus.SKIPPED_NO_CUDA, "float8 training needs CUDA", info)
    try:
        return mod.convert_to_float8_training(model), AdapterResult(AdapterStatus.OK, version=info)
    except Exception as exc:  # noqa: BLE001
        return model, AdapterResult(AdapterStatus.ERROR, f"{type(exc).__name__}: {exc}", info)
