"""Megatron-style tensor-parallel primitives.

``copy_to_tp_region`` (identity forward, all-reduce of the gradient in backward) and
``reduce_from_tp_region`` (all-reduce forward, identity backward) bracket a column-parallel /
row-parallel pair; ``shard_linear_column`` / ``shard_linear_row`` cut an ``nn.Linear`` (the row
shard keeps the bias on rank 0 only, so no rank trains a duplicate); ``sync_replicated_grads``
averages the gradients of parameters that every rank holds (embeddings, LayerNorms, LM head).
API parity: stacr/protocols/tensor_parallel.py:25-220 of the reference project.

Differences: the collective goes through ``tp_all_reduce_``, which on CUDA reduces through the
in-tree NVLink all-reduce kernels when the tensor lives in symmetric memory (the row-parallel
GEMM of ``stacr_b200.parallel.tp`` writes its partial output there) and otherwise through
``torch.distributed``; replicated gradients are synchronised as ONE flattened all-reduce instead
of one collective per parameter.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def tp_all_reduce_(tensor: torch.Tensor, group=None) -> torch.Tensor:
    """Sum ``tensor`` across the tensor-parallel group in place."""
    if _world(group) == 1:
        return tensor
    owner = getattr(tensor, "_symm_owner", None)
    if owner is not None:
        lo = (tensor.data_ptr() - owner.tensor.data_ptr()) // owner.tensor.element_size()
        owner.all_reduce_(lo, lo + tensor.numel(), average=False)
        return tensor
    dist.all_reduce(tensor, group=group)
    return tensor


class _CopyToTPRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        return tp_all_reduce_(grad, ctx.group), None


class _ReduceFromTPRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        out = x if getattr(x, "_symm_owner", None) is not None else x.clone()
        return tp_all_reduce_(out, group)

    @staticmethod
    def backward(ctx, grad):
        return grad, None


def copy_to_tp_region(input_, tp_group):
    return _CopyToTPRegion.apply(input_, tp_group)


def reduce_from_tp_region(input_, tp_group):
    return _ReduceFromTPRegion.apply(input_, tp_group)


def convert_conv1d_to_linear(model: nn.Module) -> int:
    """Swap every Conv1D (``[in, out]`` weight) for an ``nn.Linear`` with the transposed weight."""
    swapped = 0
    for name, module in list(model.named_modules()):
        if type(module).__name__ != "Conv1D":
            continue
        n_in, n_out = module.weight.shape
        bias = getattr(module, "bias", None)
        lin = nn.Linear(n_in, n_out, bias=bias is not None, device=module.weight.device, dtype=module.weight.dtype)
        with torch.no_grad():
            lin.weight.copy_(module.weight.t())
            if bias is not None:
                lin.bias.copy_(bias)
        parent_name, _, leaf = name.rpartition(".")
        setattr(model.get_submodule(parent_name) if parent_name else model, leaf, lin)
        swapped += 1
    return swapped


def _new_linear(like: nn.Linear, n_in: int, n_out: int, bias: bool) -> nn.Linear:
    return nn.Linear(n_in, n_out, bias=bias, device=like.weight.device, dtype=like.weight.dtype)


def shard_linear_column(linear: nn.Linear, tp_rank: int, tp_world_size: int) -> nn.Linear:
    """Keep output rows ``[rank * O/tp, (rank+1) * O/tp)`` (and the same slice of the bias)."""
    if linear.out_features % tp_world_size:
        raise AssertionError(f"Column shard: out_features={linear.out_features} not divisible by tp_world_size={tp_world_size}")
    size = linear.out_features // tp_world_size
    sl = slice(tp_rank * size, (tp_rank + 1) * size)
    out = _new_linear(linear, linear.in_features, size, linear.bias is not None)
    with torch.no_grad():
        out.weight.copy_(linear.weight[sl])
        if linear.bias is not None:
            out.bias.copy_(linear.bias[sl])
    return out


def shard_linear_row(linear: nn.Linear, tp_rank: int, tp_world_size: int) -> nn.Linear:
    """Keep input columns ``[rank * N/tp, (rank+1) * N/tp)``; only rank 0 keeps a bias parameter."""
    if linear.in_features % tp_world_size:
        raise AssertionError(f"Row shard: in_features={linear.in_features} not divisible by tp_world_size={tp_world_size}")
    size = linear.in_features // tp_world_size
    sl = slice(tp_rank * size, (tp_rank + 1) * size)
    keep_bias = linear.bias is not None and tp_rank == 0
    out = _new_linear(linear, size, linear.out_features, keep_bias)
    with torch.no_grad():
        out.weight.copy_(linear.weight[:, sl])
        if keep_bias:
            out.bias.copy_(linear.bias)
    return out


def replicated_parameters(model: nn.Module):
    """``(name, parameter)`` pairs that are not inside a tensor-parallel (sharded) module."""
    sharded = tuple(n + "." for n, m in model.named_modules() if type(m).__name__ in ("TPGPT2MLP", "TPGPT2Attention"))
    for name, p in model.named_parameters():
        if not name.startswith(sharded):
            yield name, p


def sync_replicated_grads(model: nn.Module, tp_group=None) -> int:
    """Average the gradients of replicated parameters with one flattened collective; returns how many tensors."""
    ws = _world(tp_group)
    grads = [p.grad for _, p in replicated_parameters(model) if p.grad is not None]
    if ws == 1 or not grads:
        return len(grads)
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=tp_group)
    flat.div_(ws)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()
    return len(grads)
