"""Linear layer that saves token-projected inputs (parity: comparators/instant/custom_op.py)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class LinearSVDOp(torch.autograd.Function):
    """``y = x Wᵀ + b`` saving ``Pᵀ x``; backward uses ``dW = Σ_b dYᵀ P (Pᵀ x)`` and ``dX = Q (Qᵀ dY W)``.

    ``pt`` is ``Pᵀ [k_x, tokens]`` and ``qt`` is ``Qᵀ [k_g, tokens]``; ``x`` is ``[batch, tokens, features]``.
    """

    @staticmethod
    def forward(ctx, x, weight, bias, pt, qt):
        ctx.save_for_backward(pt @ x, weight, pt, qt)
        ctx.has_bias = bias is not None
        return F.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        xc, weight, pt, qt = ctx.saved_tensors
        dx = qt.transpose(0, 1) @ ((qt @ dy) @ weight) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dyc = pt @ dy                                     # [batch, k_x, out]
            dw = torch.einsum("bko,bki->oi", dyc, xc)
        db = dy.sum(dim=(0, 1)) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None, None


class InstantLinear(nn.Linear):
    """``nn.Linear`` that switches to :class:`LinearSVDOp` while training, once both subspaces are set."""

    activate = True
    CompressionTensor_x = None      # P  [tokens, k_x]
    CompressionTensor_gy = None     # Q  [tokens, k_g]

    def forward(self, input):
        p, q = self.CompressionTensor_x, self.CompressionTensor_gy
        usable = (self.activate and self.training and p is not None and q is not None and input.dim() == 3
                  and input.shape[1] == p.shape[0] == q.shape[0])
        if not usable:
            return super().forward(input)
        pt = p.t().to(device=input.device, dtype=input.dtype)
        qt = q.t().to(device=input.device, dtype=input.dtype)
        return LinearSVDOp.apply(input, self.weight, self.bias, pt, qt)

    def saved_rows(self, tokens: int) -> int:
        """Rows kept per sample for backward (``tokens`` when the layer runs uncompressed)."""
        p = self.CompressionTensor_x
        return int(p.shape[1]) if (self.activate and p is not None and p.shape[0] == tokens) else int(tokens)


LinearCompressClass = InstantLinear


def wrap_linear_compression_layer(linear_layer: nn.Linear, **_unused) -> InstantLinear:
    """An :class:`InstantLinear` sharing the parameters (not copies) of ``linear_layer``."""
    new = InstantLinear(linear_layer.in_features, linear_layer.out_features, bias=linear_layer.bias is not None,
                        device="meta")
    new.weight = linear_layer.weight
    new.bias = linear_layer.bias
    new.train(linear_layer.training)
    return new


def register_filter(model: nn.Module, modules_compressed) -> nn.Module:
    """Replace each named ``nn.Linear`` by its compressing form, in place."""
    wanted = set(modules_compressed)
    for name, module in list(model.named_modules()):
        if name in wanted and isinstance(module, nn.Linear) and not isinstance(module, InstantLinear):
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, leaf, wrap_linear_compression_layer(module))
    return model
