"""Composition with block recomputation and host offload of saved tensors.

``saved_tensors_on_cpu`` differs from the reference's hook (stacr/composition.py:12-39 there) in
one deliberate way: device->host copies are issued on a dedicated copy stream and the
host->device copy in backward is prefetch-friendly (non-blocking from pinned memory), so the
offload overlaps compute instead of serialising on the current stream.  Layout (strides) of the
saved tensor is preserved, which fused attention backward kernels rely on.
Block discovery, target filtering and the checkpoint/offload wrappers follow
stacr/composition.py:42-127.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from functools import wraps

import torch
from torch import nn

_BLOCK_PATHS = (
    "transformer.h", "model.layers", "gpt_neox.layers", "bert.encoder.layer", "roberta.encoder.layer",
    "model.decoder.layers", "transformer.blocks",
)
_copy_streams: dict[int, torch.cuda.Stream] = {}


def _copy_stream(device: torch.device) -> torch.cuda.Stream:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _copy_streams:
        _copy_streams[idx] = torch.cuda.Stream(device=idx)
    return _copy_streams[idx]


def saved_tensors_on_cpu(*, pin_memory: bool = True, side_stream: bool = True):
    """Context manager: tensors saved for backward inside it live in (pinned) host memory."""

    def pack(t: torch.Tensor):
        dev = t.device
        if dev.type == "cpu":
            return dev, t.detach(), None
        if pin_memory and dev.type == "cuda" and t.layout == torch.strided:
            host = torch.empty_like(t, device="cpu", pin_memory=True, memory_format=torch.preserve_format)
            if side_stream:
                stream = _copy_stream(dev)
                stream.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(stream):
                    host.copy_(t, non_blocking=True)
                    done = torch.cuda.Event()
                    done.record(stream)
                t.record_stream(stream)
                return dev, host, done
            host.copy_(t)
            return dev, host, None
        return dev, t.detach().cpu(), None

    def unpack(record):
        dev, host, done = record
        if done is not None:
            done.synchronize()  # the device->host copy must have landed before it is read back
        pinned = host.layout == torch.strided and host.is_pinned()
        return host.to(dev, non_blocking=pinned)

    return torch.autograd.graph.saved_tensors_hooks(pack, unpack)


def transformer_blocks(model: nn.Module) -> list[nn.Module]:
    """The block stack of common decoder/encoder layouts; pass blocks explicitly for anything else."""
    for path in _BLOCK_PATHS:
        try:
            stack = model.get_submodule(path)
        except AttributeError:
            continue
        if isinstance(stack, (nn.ModuleList, nn.Sequential)):
            return list(stack)
    raise ValueError("Cannot locate transformer blocks; pass your block sequence explicitly.")


def block_target_names(model: nn.Module, blocks: Sequence[nn.Module], predicate: Callable[[int], bool], **selection) -> list[str]:
    """Selected projection names that live inside the blocks whose index satisfies ``predicate``."""
    from .surgery import select_target_names

    inside = {id(m) for i, blk in enumerate(blocks) if predicate(i) for m in blk.modules()}
    return [n for n in select_target_names(model, **selection) if id(model.get_submodule(n)) in inside]


def _checked(blocks, indices) -> list[int]:
    chosen = sorted(set(indices))
    for i in chosen:
        if not isinstance(i, int) or isinstance(i, bool) or not 0 <= i < len(blocks):
            raise ValueError(f"Block indices must be integers in [0, {len(blocks)})")
    return chosen


def _wrap_forward(block: nn.Module, marker: str, what: str, index: int, make):
    if hasattr(block, marker):
        raise ValueError(f"Block {index} already has {what} enabled")
    inner = block.forward
    setattr(block, marker, inner)
    block.forward = wraps(inner)(make(inner))


def checkpoint_blocks(blocks: Sequence[nn.Module], indices: Sequence[int]) -> list[int]:
    """Non-reentrant activation checkpointing (RNG preserved) with compression-state replay."""
    from .adaptive_checkpointing import checkpoint

    chosen = _checked(blocks, indices)
    for i in chosen:
        def make(inner):
            def forward(*args, **kwargs):
                if not torch.is_grad_enabled():
                    return inner(*args, **kwargs)
                return checkpoint(inner, *args, use_reentrant=False, preserve_rng_state=True, **kwargs)
            return forward
        _wrap_forward(blocks[i], "_stacr_checkpoint_forward", "checkpointing", i, make)
    return chosen


def offload_blocks(blocks: Sequence[nn.Module], indices: Sequence[int], *, pin_memory: bool = True) -> list[int]:
    """Keep the saved tensors of the chosen blocks in host memory until backward needs them."""
    chosen = _checked(blocks, indices)
    for i in chosen:
        def make(inner):
            def forward(*args, **kwargs):
                with saved_tensors_on_cpu(pin_memory=pin_memory):
                    return inner(*args, **kwargs)
            return forward
        _wrap_forward(blocks[i], "_stacr_offload_forward", "CPU offload", i, make)
    return chosen
