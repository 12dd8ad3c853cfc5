"""PRAC-linear comparator: save a random projection ``x P`` of the layer input instead of ``x``.

``P`` has iid ``N(0, 1/r)`` entries, so ``E[P P^T] = I`` and ``dW = (dY^T (x P)) P^T`` is an unbiased estimate
of the weight gradient.  ``P`` is resampled every ``update_proj_gap`` steps from a seed derived with SHA-256
from ``(seed_base, layer name, window index)`` so it is identical across processes and platforms.
Parity: stacr/protocols/prac.py:49-386 of the reference project.
"""

from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn
from torch.nn import functional as F


@dataclass
class PRACConfig:
    rank: int = 8
    update_proj_gap: int = 50
    proj_dtype: Optional[str] = None
    seed_base: int = 42
    quiet: bool = False


def _resolve_proj_dtype(spec: Optional[str]) -> torch.dtype:
    table = {None: torch.float32, "float32": torch.float32, "fp32": torch.float32, "float16": torch.float16, "fp16": torch.float16,
             "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
    if spec not in table:
        raise ValueError(f"Unknown proj_dtype: {spec!r}")
    return table[spec]


def _layer_seed(seed_base: int, layer_name: str, window_idx: int) -> int:
    digest = hashlib.sha256(f"{int(seed_base)}:{layer_name}:{int(window_idx)}".encode("utf-8")).digest()
    return int.from_bytes(digest[:4], byteorder="big", signed=False)


def _is_hf_conv1d(module: nn.Module) -> bool:
    return type(module).__name__ == "Conv1D" and hasattr(module, "weight")


class PRACFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_tensor, weight, bias, projection):
        flat = input_tensor.reshape(-1, input_tensor.shape[-1])
        p = projection if projection.dtype == flat.dtype else projection.to(flat.dtype)
        ctx.save_for_backward(flat @ p, p, weight)
        ctx.input_shape, ctx.has_bias = tuple(input_tensor.shape), bias is not None
        return F.linear(input_tensor, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        x_proj, p, weight = ctx.saved_tensors
        g = grad_output.reshape(-1, weight.shape[0])
        grad_weight = ((g.float().t() @ x_proj.float()) @ p.float().t()).to(weight.dtype)
        grad_input = (g @ weight.to(g.dtype)).reshape(ctx.input_shape)
        return grad_input, grad_weight, (g.sum(0) if ctx.has_bias else None), None


class PRACLinear(nn.Module):
    def __init__(self, linear: nn.Linear, config: PRACConfig, layer_name: str = ""):
        super().__init__()
        self.linear, self.config, self.layer_name = linear, config, layer_name
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.effective_rank = max(1, min(int(config.rank), self.in_features))
        self.proj_dtype = _resolve_proj_dtype(config.proj_dtype)
        self.register_buffer("step_counter", torch.zeros((), dtype=torch.int64, device=linear.weight.device))
        self._last_window_idx = 0
        self.register_buffer("projection", self._sample_projection(0, linear.weight.device, self.proj_dtype))

    def _sample_projection(self, step: int, device=None, dtype=None) -> torch.Tensor:
        window = int(step) // max(1, int(self.config.update_proj_gap))
        gen = torch.Generator(device="cpu").manual_seed(_layer_seed(self.config.seed_base, self.layer_name, window))
        p = torch.randn(self.in_features, self.effective_rank, generator=gen, dtype=torch.float32) / math.sqrt(self.effective_rank)
        return p.to(device=device if device is not None else self.linear.weight.device, dtype=dtype or self.proj_dtype)

    def set_global_step(self, step: int) -> None:
        step = int(step)
        self.step_counter.fill_(step)
        window = step // max(1, int(self.config.update_proj_gap))
        if window != self._last_window_idx:
            self._last_window_idx = window
            self.projection.copy_(self._sample_projection(step, self.projection.device, self.projection.dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if getattr(self, "_disable_prac_compression", False) or not (self.training and torch.is_grad_enabled()):
            return self.linear(x)
        return PRACFunction.apply(x, self.linear.weight, self.linear.bias, self.projection)

    def projection_buffer_bytes(self) -> int:
        return self.projection.numel() * self.projection.element_size()

    def saved_activation_bytes(self, batch_tokens: int, act_dtype: torch.dtype) -> int:
        width = torch.empty((), dtype=act_dtype).element_size()
        cast = self.projection.numel() * width if act_dtype != self.projection.dtype else 0
        return batch_tokens * self.effective_rank * width + cast


def set_prac_global_step(model: nn.Module, step: int) -> None:
    for m in model.modules():
        if isinstance(m, PRACLinear):
            m.set_global_step(step)


def replace_linear_with_prac(model: nn.Module, target_names, config: PRACConfig | None = None) -> list[PRACLinear]:
    """Wrap the named ``nn.Linear`` modules (Conv1D is converted to Linear first)."""
    config = config or PRACConfig()
    out = []
    for name in target_names:
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        module = getattr(parent, leaf)
        if _is_hf_conv1d(module):
            lin = nn.Linear(module.weight.shape[0], module.weight.shape[1], bias=module.bias is not None,
                            device=module.weight.device, dtype=module.weight.dtype)
            with torch.no_grad():
                lin.weight.copy_(module.weight.t())
                if module.bias is not None:
                    lin.bias.copy_(module.bias)
            module = lin
        if not isinstance(module, nn.Linear):
            raise TypeError(f"{name} is not a linear projection")
        wrapped = PRACLinear(module, config, layer_name=name)
        setattr(parent, leaf, wrapped)
        out.append(wrapped)
    if not config.quiet:
        print(f"[PRAC] wrapped {len(out)} layers at rank {config.rank}")
    return out


def prac_stored_bytes_per_layer(batch_tokens: int, in_features: int, rank: int, act_dtype=torch.float16, proj_dtype=torch.float16) -> dict:
    width = torch.empty((), dtype=act_dtype).element_size()
    r = min(rank, in_features)
    return {"saved_projection_bytes": batch_tokens * r * width,
            "projection_buffer_bytes": in_features * r * torch.empty((), dtype=proj_dtype).element_size(),
            "dense_bytes": batch_tokens * in_features * width}
