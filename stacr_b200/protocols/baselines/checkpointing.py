"""Activation-checkpointing baseline modes and the replay guard around ``torch.utils.checkpoint``.

``apply_checkpointing(model, mode)`` with ``mode`` in ``none | auto | transformer_hf | vision_stage | vision_block |
attention_only``.  Every checkpoint issued through this module carries the compression replay contexts, so layers
compressed inside a checkpointed region see the same basis and budget on recomputation.  Unlike the reference
(stacr/protocols/baselines/checkpointing.py:164-224 there), nothing is monkey-patched at import time: the guard is
installed explicitly by ``install_checkpoint_guard()`` (idempotent, reversible) or implicitly by ``apply_checkpointing``.
"""

from __future__ import annotations

import warnings
from contextlib import contextmanager

import torch
import torch.utils.checkpoint as _tuc
from torch import nn

from ...adaptive_checkpointing import RecomputationGuard, checkpoint_contexts, get_global_recomputation_guard  # noqa: F401

_ORIGINAL = None


def _checkpoint_with_guard(function, *args, **kwargs):
    """Non-reentrant checkpoint with the replay contexts; a C1-registered site goes through the boundary codec."""
    from ..checkpointing import get_active_c1_runtime, stacr_checkpoint

    runtime = get_active_c1_runtime()
    if runtime is not None:
        codec = runtime.resolve_site(function)
        if codec is not None and args and isinstance(args[0], torch.Tensor):
            try:
                return stacr_checkpoint(function, *args, codec=codec, **{k: v for k, v in kwargs.items() if k not in ("use_reentrant", "preserve_rng_state", "context_fn", "determinism_check", "debug")})
            except Exception as exc:  # noqa: BLE001 - fall back to the plain checkpoint, once, loudly
                warnings.warn(f"C1 boundary compression failed for a site, using a plain checkpoint: {exc}")
    kwargs.pop("use_reentrant", None)
    kwargs.setdefault("context_fn", checkpoint_contexts)
    base = _ORIGINAL or _tuc.checkpoint
    return base(function, *args, use_reentrant=False, **kwargs)


def install_checkpoint_guard() -> None:
    """Route ``torch.utils.checkpoint.checkpoint`` through the guard (so library-issued checkpoints replay state too)."""
    global _ORIGINAL
    if _ORIGINAL is None:
        _ORIGINAL = _tuc.checkpoint
        _tuc.checkpoint = _checkpoint_with_guard


def uninstall_checkpoint_guard() -> None:
    global _ORIGINAL
    if _ORIGINAL is not None:
        _tuc.checkpoint = _ORIGINAL
        _ORIGINAL = None


def _wrap(module: nn.Module, marker: str = "_baseline_ckpt_forward") -> bool:
    if hasattr(module, marker):
        return False
    inner = module.forward

    def forward(*args, **kwargs):
        if not (torch.is_grad_enabled() and module.training):
            return inner(*args, **kwargs)
        return _checkpoint_with_guard(inner, *args, **kwargs)

    setattr(module, marker, inner)
    module.forward = forward
    return True


def _unwrap(module: nn.Module, marker: str = "_baseline_ckpt_forward") -> None:
    if hasattr(module, marker):
        module.forward = getattr(module, marker)
        delattr(module, marker)


def _transformer_blocks(model):
    from ...composition import transformer_blocks

    return transformer_blocks(model)


def _attention_modules(model):
    return [m for n, m in model.named_modules() if n.split(".")[-1] in ("attn", "attention", "self_attn", "self_attention")]


def _vision_stages(model):
    for attr in ("layer1", "layer2", "layer3", "layer4"):
        if hasattr(model, attr):
            yield getattr(model, attr)
    for attr in ("stages", "features"):
        stack = getattr(model, attr, None)
        if isinstance(stack, (nn.Sequential, nn.ModuleList)):
            yield from stack


def apply_checkpointing(model: nn.Module, mode: str) -> int:
    """Enable a checkpointing mode in place; returns how many modules were wrapped."""
    mode = str(mode).lower()
    if mode == "none":
        return 0
    if mode in ("auto", "transformer_hf"):
        if hasattr(model, "gradient_checkpointing_enable"):
            install_checkpoint_guard()
            model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
            return len(_transformer_blocks(model))
        return sum(_wrap(b) for b in _transformer_blocks(model))
    if mode == "attention_only":
        return sum(_wrap(m) for m in _attention_modules(model))
    if mode == "vision_stage":
        return sum(_wrap(s) for s in _vision_stages(model))
    if mode == "vision_block":
        return sum(_wrap(b) for s in _vision_stages(model) for b in (s if isinstance(s, (nn.Sequential, nn.ModuleList)) else [s]))
    raise ValueError(f"Unknown checkpointing mode: {mode!r}")


def disable_checkpointing(model: nn.Module, mode: str) -> None:
    if str(mode).lower() in ("auto", "transformer_hf") and hasattr(model, "gradient_checkpointing_disable"):
        model.gradient_checkpointing_disable()
    for m in model.modules():
        _unwrap(m)


@contextmanager
def checkpointing_context(model: nn.Module, mode: str):
    apply_checkpointing(model, mode)
    try:
        yield model
    finally:
        disable_checkpointing(model, mode)
