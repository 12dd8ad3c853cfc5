"""Linear layer whose saved input is an SVD / TT / Tucker factorisation (comparators for the STAC-R layer).

Forward is the exact linear; what is saved for backward are the factors of the input batch.  SVD factors are
contracted natively, ``dW = ((dY^T U) diag(s)) V^T``; TT and Tucker are reconstructed in backward (their
contraction order depends on the tensorisation).  Parity: stacr/protocols/layers.py:7-352 of the reference project.
"""

from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

from .compression import Compressor


class CompressedFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_tensor, weight, bias, config):
        flat = input_tensor.reshape(-1, input_tensor.shape[-1])
        out = F.linear(input_tensor, weight, bias)
        method = config.get("method", "svd")
        bits = config.get("quantize_bits")
        with torch.no_grad():
            if method == "svd":
                factors = Compressor.compress_svd_factors(flat, config.get("rank", 8), use_lowrank=config.get("use_lowrank", False))
                packed = Compressor.quantize_svd_factors(factors, bits) if bits else factors
            elif method == "tt":
                factors = Compressor.compress_tt_factors(flat, config["reshape_shape"], config.get("rank", 8))
                packed = Compressor.quantize_tt_factors(factors, bits) if bits else factors
            elif method == "tucker":
                factors = Compressor.compress_tucker_factors(flat, config["reshape_shape"], config["ranks"])
                packed = Compressor.quantize_tucker_factors(factors, bits) if bits else factors
            else:
                raise ValueError(f"Unknown compression method {method!r}")
        ctx.packed, ctx.method, ctx.bits = packed, method, bits
        ctx.save_for_backward(weight)
        ctx.input_shape, ctx.input_dtype, ctx.has_bias = tuple(input_tensor.shape), input_tensor.dtype, bias is not None
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (weight,) = ctx.saved_tensors
        g = grad_output.reshape(-1, weight.shape[0])
        grad_input = (g @ weight.to(g.dtype)).reshape(ctx.input_shape) if ctx.needs_input_grad[0] else None
        grad_weight = None
        if ctx.needs_input_grad[1]:
            gf = g.float()
            if ctx.method == "svd":
                u, s, vh = Compressor.dequantize_svd_factors(ctx.packed) if ctx.bits else ctx.packed
                grad_weight = ((gf.t() @ u.float()) * s.float()) @ vh.float()  # factor-native
            elif ctx.method == "tt":
                x = Compressor.decompress_tt(Compressor.dequantize_tt_factors(ctx.packed) if ctx.bits else ctx.packed)
                grad_weight = gf.t() @ x.float().reshape(gf.shape[0], -1)
            else:
                x = Compressor.decompress_tucker(Compressor.dequantize_tucker_factors(ctx.packed) if ctx.bits else ctx.packed)
                grad_weight = gf.t() @ x.float().reshape(gf.shape[0], -1)
            grad_weight = grad_weight.to(weight.dtype)
        grad_bias = g.sum(0) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return grad_input, grad_weight, grad_bias, None


class CompressedLinear(nn.Module):
    """``nn.Linear`` drop-in; ``compression_config`` = ``{"method": "svd"|"tt"|"tucker", "rank"/"ranks", "reshape_shape", "quantize_bits"}``."""

    def __init__(self, in_features, out_features, compression_config, bias=True):
        super().__init__()
        self._validate_config(in_features, compression_config)
        self.linear = nn.Linear(in_features, out_features, bias=bias)
        self.config = dict(compression_config)

    @classmethod
    def from_linear(cls, module: nn.Linear, compression_config) -> "CompressedLinear":
        new = cls(module.in_features, module.out_features, compression_config, bias=module.bias is not None)
        new.linear = module
        new.train(module.training)
        return new

    def forward(self, x):
        if not (self.training and torch.is_grad_enabled() and self.linear.weight.requires_grad):
            return self.linear(x)
        return CompressedFunction.apply(x, self.linear.weight, self.linear.bias, self.config)

    @staticmethod
    def _validate_config(in_features: int, config):
        method = config.get("method", "svd")
        if method not in ("svd", "tt", "tucker"):
            raise ValueError(f"Unknown compression method {method!r}")
        if method in ("tt", "tucker") and "reshape_shape" not in config:
            raise ValueError(f"{method} needs reshape_shape")
        if method == "tucker" and "ranks" not in config:
            raise ValueError("tucker needs ranks")
        if config.get("quantize_bits") not in (None, 0, 4, 8):
            raise ValueError("quantize_bits must be None, 4 or 8")
