"""Adapter around optional ``torchao`` low-bit optimizers / float8 training (graceful skip when absent).

Parity: stacr/protocols/baselines/torchao_adapter.py of the reference project.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._optional import AdapterResult, AdapterStatus, final_json, probe

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


TORCHAO_MODES = ("auto", "int8", "fp8")


def get_torchao_version() -> Optional[str]:
    ok, info, _ = probe("torchao")
    return info if ok else None


def _quantize(model: torch.nn.Module, mode: str):
    """Apply torchao's weight quantisation in place; returns the mode that was applied."""
    found, err, q = probe("torchao.quantization")
    if not found or not hasattr(q, "quantize_"):
        raise RuntimeError(f"torchao.quantization.quantize_ unavailable: {err}")
    if mode in ("auto", "fp8"):
        maker = getattr(q, "float8_dynamic_activation_float8_weight", None) or getattr(q, "Float8DynamicActivationFloat8WeightConfig", None)
        if maker is not None and hasattr(torch, "float8_e4m3fn"):
            q.quantize_(model, maker())
            return "fp8"
        if mode == "fp8":
            raise RuntimeError("this torchao build has no float8 dynamic quantisation")
    maker = getattr(q, "int8_dynamic_activation_int8_weight", None) or getattr(q, "Int8DynamicActivationInt8WeightConfig", None)
    if maker is None:
        raise RuntimeError("this torchao build has no int8 dynamic quantisation")
    q.quantize_(model, maker())
    return "int8"


def try_enable_torchao(model: torch.nn.Module, mode: str = "auto"):
    """Quantise the model's linears with torchao (``auto`` prefers float8 and falls back to int8); ``(model, result)``."""
    if mode not in TORCHAO_MODES:
        return model, AdapterResult(AdapterStatus.ERROR, f"Invalid mode {mode!r}. Valid: {TORCHAO_MODES}")
    if not torch.cuda.is_available():
        return model, AdapterResult(AdapterStatus.SKIPPED_NO_CUDA, "the torchao baseline needs CUDA", details={"requested_mode": mode})
    ok, info, _ = probe("torchao")
    if not ok:
        return model, AdapterResult(AdapterStatus.SKIPPED_NOT_INSTALLED, str(info), details={"requested_mode": mode})
    tried = [mode] + (["int8"] if mode == "auto" else [])
    errors = []
    for attempt in tried:
        try:
            applied = _quantize(model, attempt)
            return model, AdapterResult(AdapterStatus.OK, f"torchao enabled ({applied})", info,
                                        {"requested_mode": mode, "applied_mode": applied, **({"fallback_reason": errors[0]} if errors else {})})
        except Exception as exc:  # noqa: BLE001
            errors.append(f"{type(exc).__name__}: {exc}")
    return model, AdapterResult(AdapterStatus.ERROR, "; ".join(errors), info, {"requested_mode": mode})


def create_torchao_final_json(result: AdapterResult, output_dir: str) -> dict:
    return final_json("torchao", result, output_dir)
