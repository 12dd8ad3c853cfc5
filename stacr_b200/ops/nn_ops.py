"""Normalisation, activation and loss ops of the model zoo.

For bf16 CUDA tensors these dispatch to the sm_100a kernels in ``csrc/nn_kernels.cu`` (fused
LayerNorm forward/backward with fp32 statistics, GELU forward/backward, fused softmax
cross-entropy that writes the logit gradient in place of a second pass).  Everything else uses
the framework ops, which are also the oracles of the kernel tests.
"""

from __future__ import annotations

import torch
from torch.nn import functional as F

from . import _lib


def _kernel_tensor(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


# ------------------------------------------------------------------------------ LayerNorm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        from . import nn_kernels

        x2d = x.reshape(-1, x.shape[-1]).contiguous()
        y, mean, rstd = nn_kernels.layernorm_fwd(x2d, weight, bias, eps)
        ctx.save_for_backward(x2d, weight, mean, rstd)
        ctx.has_bias = bias is not None
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        from . import nn_kernels

        x2d, weight, mean, rstd = ctx.saved_tensors
        dy2d = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx, dw, db = nn_kernels.layernorm_bwd(dy2d, x2d, weight, mean, rstd)
        return dx.reshape(dy.shape), dw.to(weight.dtype), (db.to(weight.dtype) if ctx.has_bias else None), None


def layer_norm(x, weight, bias, eps: float = 1e-5):
    if _kernel_tensor(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _LayerNormFn.apply(x, weight, bias, eps)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


class _ParallelNormsFn(torch.autograd.Function):
    """``(LN1(x), LN2(x), x)`` for a parallel-residual block ``x + f(LN1(x)) + g(LN2(x))``.

    Forward reads ``x`` once for both normalisations.  The third output is ``x`` itself, handed on to the residual sum,
    so that all three gradient streams that meet at ``x`` arrive in this function's backward, which forms
    ``LNbwd(g1) + LNbwd(g2) + g3`` in one kernel instead of two normalisation backwards and two accumulating adds.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, eps):
        from . import nn_kernels

        x2d = x.reshape(-1, x.shape[-1]).contiguous()
        y1, y2, mean, rstd = nn_kernels.layernorm_fwd2(x2d, w1, b1, w2, b2, eps)
        ctx.save_for_backward(x2d, w1, w2, mean, rstd)
        ctx.x_shape = x.shape
        return y1.reshape(x.shape), y2.reshape(x.shape), x.view_as(x)

    @staticmethod
    def backward(ctx, g1, g2, g3):
        from . import nn_kernels

        x2d, w1, w2, mean, rstd = ctx.saved_tensors

        def flat(g):
            return None if g is None else g.reshape(x2d.shape).to(torch.bfloat16).contiguous()

        g1, g2, g3 = flat(g1), flat(g2), flat(g3)
        if g1 is None:
            g1 = torch.zeros_like(x2d)
        if g2 is None:
            g2 = torch.zeros_like(x2d)
        dx, dw1, db1, dw2, db2 = nn_kernels.layernorm_bwd2(g1, g2, g3, x2d, w1, w2, mean, rstd)
        return dx.reshape(ctx.x_shape), dw1.to(w1.dtype), db1.to(w1.dtype), dw2.to(w2.dtype), db2.to(w2.dtype), None


def parallel_norms_supported(x, w1, b1, w2, b2) -> bool:
    return (_kernel_tensor(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 2048 and b1 is not None and b2 is not None
            and w1.shape == w2.shape)


def parallel_layer_norms(x, w1, b1, w2, b2, eps: float = 1e-5):
    """``(LN(x; w1, b1), LN(x; w2, b2), x)``: use the third result as the residual operand (see ``_ParallelNormsFn``)."""
    return _ParallelNormsFn.apply(x, w1, b1, w2, b2, eps)


class _Add3Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, c):
        from . import nn_kernels

        return nn_kernels.add3(a.contiguous(), b.contiguous(), c.contiguous())

    @staticmethod
    def backward(ctx, g):
        return g, g, g


def add3(a, b, c):
    """``a + b + c`` in one pass for bf16 CUDA tensors of one shape."""
    if _kernel_tensor(a) and a.shape == b.shape == c.shape and b.dtype == c.dtype == a.dtype and a.numel() % 8 == 0:
        return _Add3Fn.apply(a, b, c)
    return a + b + c


# ------------------------------------------------------------------------------ column sums handed from producer to consumer
class _ColumnSums:
    """Column sums of a gradient matrix that some kernel produced as a by-product, offered to whoever needs them next.

    The backward of an activation writes ``dX`` and can sum its columns on the way; the backward of the linear layer that
    fed the activation runs next and needs exactly those sums for its bias gradient.  The two are separate autograd nodes,
    so the sums travel through this mailbox keyed by the matrix's storage address, shape and version.  The mailbox keeps
    the matrix itself alive while its entry exists, so the address cannot be recycled for another tensor and a match is
    never a coincidence.  Two slots: ``offered`` holds a producer's by-product and is emptied when it is taken;
    ``remembered`` holds sums that ``bias_grad`` computed itself and stays until the next such computation, so that two
    layers that receive the same gradient tensor (the attention output projection and the MLP output projection of a
    parallel-residual block, whose backward passes are separated by the whole MLP) sum it once.  A lookup that matches
    neither slot leaves the caller to compute the sums.
    """

    def __init__(self):
        self.offered = None        # (key, sums, matrix)
        self.remembered = None

    @staticmethod
    def _key(t: torch.Tensor, cols: int):
        return (t.data_ptr(), t.numel(), cols, t._version, t.device.index)

    def offer(self, matrix: torch.Tensor, sums: torch.Tensor, single_use: bool) -> None:
        entry = (self._key(matrix, sums.numel()), sums, matrix)
        if single_use:
            self.offered = entry
        else:
            self.remembered = entry

    def take(self, matrix: torch.Tensor, cols: int):
        key = self._key(matrix, cols)
        if self.offered is not None and self.offered[0] == key:
            sums, self.offered = self.offered[1], None
            return sums
        if self.remembered is not None and self.remembered[0] == key:
            return self.remembered[1]
        return None

    def clear(self) -> None:
        self.offered = self.remembered = None


column_sums = _ColumnSums()


def bias_grad(g2d: torch.Tensor) -> torch.Tensor:
    """fp32 column sums of a bf16 gradient matrix ``[rows, out]``: taken from the mailbox when its producer left them there."""
    from . import stacr_ops

    hit = column_sums.take(g2d, g2d.shape[1])
    if hit is not None:
        return hit
    sums = stacr_ops.colsum(g2d)
    column_sums.offer(g2d, sums, single_use=False)
    return sums


# ------------------------------------------------------------------------------ GELU
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tanh_form: bool):
        from . import nn_kernels

        xc = x.contiguous()
        ctx.save_for_backward(xc)
        ctx.tanh_form = tanh_form
        return nn_kernels.gelu_fwd(xc, tanh_form)

    @staticmethod
    def backward(ctx, dy):
        from . import nn_kernels

        (x,) = ctx.saved_tensors
        if x.dim() >= 2 and x.shape[-1] % 8 == 0:
            dx, sums = nn_kernels.gelu_bwd_colsum(dy.contiguous(), x, ctx.tanh_form)
            column_sums.offer(dx, sums, single_use=True)      # the bias gradient of the projection that produced x
            return dx, None
        return nn_kernels.gelu_bwd(dy.contiguous(), x, ctx.tanh_form), None


def gelu(x, approximate: str = "none"):
    if _kernel_tensor(x) and x.numel() % 8 == 0:
        return _GeluFn.apply(x, approximate == "tanh")
    return F.gelu(x, approximate=approximate)


# ------------------------------------------------------------------------------ cross-entropy
class _CrossEntropyFn(torch.autograd.Function):
    """Mean cross-entropy over rows with ``target != -100``.  Forward reads the logits once (loss and row log-sum-exp);
    backward reads them once more and writes the gradient with the upstream scalar folded in."""

    @staticmethod
    def forward(ctx, logits, target):
        from . import nn_kernels

        logits = logits.contiguous()
        loss, tgt, lse, inv_valid = nn_kernels.cross_entropy_fwd(logits, target.contiguous())
        ctx.save_for_backward(logits, tgt, lse, inv_valid)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        from . import nn_kernels

        logits, tgt, lse, inv_valid = ctx.saved_tensors
        return nn_kernels.cross_entropy_bwd(logits, tgt, lse, inv_valid, dloss), None


def cross_entropy(logits, target):
    if _kernel_tensor(logits) and logits.shape[-1] % 8 == 0:
        return _CrossEntropyFn.apply(logits, target)
    return F.cross_entropy(logits.float(), target, ignore_index=-100)


class _PaddedHeadCEFn(torch.autograd.Function):
    """``cross_entropy(hidden @ weight^T, target)`` for a vocabulary that is not a multiple of 8 (GPT-2: 50257).

    Library GEMMs fall back to unaligned legacy kernels when the logits' leading dimension is odd, and the loss kernel needs
    16-byte rows.  Here the logits live in a buffer whose rows are padded to a multiple of 64 columns: the in-tree GEMM writes
    the first ``V`` columns (its output takes a leading dimension), the padding holds a large negative value so that it gets
    no probability, and both backward products read the same padded buffer through strided views.
    """

    @staticmethod
    def forward(ctx, hidden, weight, target):
        from . import nn_kernels
        from .gemm import gemm

        rows, v = hidden.shape[0], weight.shape[0]
        vp = (v + 63) // 64 * 64
        h = hidden if hidden.dtype == torch.bfloat16 else hidden.to(torch.bfloat16)
        h = h.contiguous()
        w = weight.detach().to(torch.bfloat16).contiguous()
        logits = torch.empty(rows, vp, dtype=torch.bfloat16, device=hidden.device)
        logits[:, v:].fill_(-30000.0)
        gemm(h, w, out=logits[:, :v])
        loss, tgt, lse, inv_valid = nn_kernels.cross_entropy_fwd(logits, target.contiguous())
        ctx.save_for_backward(h, w, logits, tgt, lse, inv_valid)
        ctx.v, ctx.hidden_dtype, ctx.weight_dtype = v, hidden.dtype, weight.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        from . import nn_kernels
        from .gemm import gemm

        h, w, logits, tgt, lse, inv_valid = ctx.saved_tensors
        d = nn_kernels.cross_entropy_bwd(logits, tgt, lse, inv_valid, dloss)[:, :ctx.v]      # [rows, V] view, rows padded
        dh = gemm(d, w, b_mn=True).to(ctx.hidden_dtype) if ctx.needs_input_grad[0] else None
        dw = gemm(d, h, a_mn=True, b_mn=True, out_dtype=torch.float32).to(ctx.weight_dtype) if ctx.needs_input_grad[1] else None
        return dh, dw, None


def linear_cross_entropy(hidden, weight, target, chunk: int = 0):
    """``cross_entropy(hidden @ weight^T, target)`` evaluated in row chunks to bound the logits workspace."""
    from . import _lib

    padded = hidden.is_cuda and weight.shape[0] % 8 != 0 and hidden.shape[-1] % 8 == 0 and _lib.available() and \
        (hidden.dtype == torch.bfloat16 or torch.is_autocast_enabled())
    if padded:
        def head(h, t):
            return _PaddedHeadCEFn.apply(h, weight, t)
    else:
        def head(h, t):
            return cross_entropy(linear(h, weight), t)
    if not chunk or hidden.shape[0] <= chunk:
        return head(hidden, target)
    valid = (target != -100).sum().clamp_min(1)
    total = hidden.new_zeros((), dtype=torch.float32)
    for lo in range(0, hidden.shape[0], chunk):
        t = target[lo:lo + chunk]
        n = (t != -100).sum()
        total = total + head(hidden[lo:lo + chunk], t).float() * n
    return total / valid


# ------------------------------------------------------------------------------ plain linear layer
class _LinearFn(torch.autograd.Function):
    """``y = x W^T + b`` for a projection that is not compressed.

    All three products run on the in-tree tcgen05 GEMM on bf16 operands (the bf16 copy of the weight is the shadow the
    fused optimizer keeps current, when there is one): forward ``X W^T + b`` with the bias added in the epilogue, the input
    gradient ``dY W`` reading ``W[out, in]`` as an MN-major operand (no transpose is materialised), and the weight gradient
    ``dY^T X`` with fp32 accumulation *and fp32 output*: under autocast a library path produces a bf16 ``dW``, casts it to
    fp32 and, with a flat gradient buffer, copies it into its slot; here the kernel writes fp32 once, straight into the
    slot when a gradient synchroniser has lent one (``weight._sb_grad_out``).
    """

    @staticmethod
    def forward(ctx, x2d, weight, bias):
        # 2-D in, 2-D out: the caller reshapes outside, so that the output is not a view made inside the function
        # (the fused-QKV rotary embedding modifies it in place)
        from ..layers import _bf16_weight

        from .gemm import gemm

        xa = (x2d if x2d.dtype == torch.bfloat16 else x2d.to(torch.bfloat16)).contiguous()
        wb = _bf16_weight(weight).contiguous()
        y = gemm(xa, wb, bias=None if bias is None else bias.detach().float().contiguous())
        ctx.save_for_backward(xa, weight)
        ctx.in_dtype, ctx.bias_dtype = x2d.dtype, None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..layers import _bf16_weight
        from . import stacr_ops
        from .gemm import gemm

        xa, weight = ctx.saved_tensors
        out_features, in_features = weight.shape
        g = (dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(g, _bf16_weight(weight).contiguous(), b_mn=True).to(ctx.in_dtype)
        if ctx.needs_input_grad[1]:
            slot = getattr(weight, "_sb_grad_out", None) if getattr(weight, "_sb_grad_fresh", False) else None
            if slot is not None and slot.dtype == torch.float32 and weight.dtype == torch.float32:
                weight._sb_grad_fresh = False
            else:
                slot = None
            dw = gemm(g, xa, a_mn=True, b_mn=True, out=slot, out_dtype=torch.float32)
            ready = getattr(weight, "_sb_grad_ready", None) if slot is not None else None
            if ready is not None and not getattr(weight, "_sb_tied", False):
                ready()      # the slot is the gradient: nothing goes back through autograd (it would be cloned)
                dw = None
            elif dw.dtype != weight.dtype:
                dw = dw.to(weight.dtype)
        if ctx.bias_dtype is not None and ctx.needs_input_grad[2]:
            db = bias_grad(g).to(ctx.bias_dtype)
        return dx, dw, db


def linear(x, weight, bias=None):
    """Linear map with the fp32-direct weight gradient on a B200 when the activations are (or autocast makes them) bf16."""
    usable = (x.is_cuda and weight.is_cuda and weight.dim() == 2 and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 and x.numel() > 0
              and _lib.available()
              and (x.dtype == torch.bfloat16 or (torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16))
              and torch.is_grad_enabled() and weight.requires_grad)
    if usable:
        y = _LinearFn.apply(x.reshape(-1, x.shape[-1]) if x.dim() != 2 else x, weight, bias)
        return y if x.dim() == 2 else y.reshape(*x.shape[:-1], weight.shape[0])
    return F.linear(x, weight, bias)


# ------------------------------------------------------------------------------ token embedding
class _EmbeddingFn(torch.autograd.Function):
    """bf16 rows of an embedding table; the table's fp32 gradient is scatter-added by an in-tree kernel, straight into the
    slot a gradient synchroniser has lent when there is one.  The rows are read from the optimizer's bf16 copy of the table
    when it exists (what a cast of the fp32 rows would give, without touching the fp32 table)."""

    @staticmethod
    def forward(ctx, weight, ids, padding_idx):
        from ..layers import _bf16_weight
        from . import nn_kernels

        table = _bf16_weight(weight) if getattr(weight, "_bf16_shadow", None) is not None else weight.detach()
        ctx.save_for_backward(ids)
        ctx.weight, ctx.padding_idx = weight, padding_idx
        return nn_kernels.embedding_fwd(table.contiguous(), ids)

    @staticmethod
    def backward(ctx, dy):
        from . import nn_kernels

        (ids,) = ctx.saved_tensors
        weight = ctx.weight
        slot = getattr(weight, "_sb_grad_out", None) if getattr(weight, "_sb_grad_fresh", False) else None
        if slot is not None and slot.dtype == torch.float32 and weight.dtype == torch.float32 and not getattr(weight, "_sb_tied", False):
            weight._sb_grad_fresh = False
        else:
            slot = None
        g = (dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16))
        dw = nn_kernels.embedding_bwd(g, ids, weight.shape[0], ctx.padding_idx, out=slot)
        ready = getattr(weight, "_sb_grad_ready", None) if slot is not None else None
        if ready is not None:
            ready()
            return None, None, None
        return dw.to(weight.dtype), None, None


def embedding(ids, weight, padding_idx=None):
    """Token embedding lookup producing bf16 on a B200 under bf16 autocast (see ``_EmbeddingFn``); the stock op elsewhere."""
    usable = (weight.is_cuda and ids.is_cuda and weight.dim() == 2 and weight.shape[1] % 8 == 0 and _lib.available() and ids.numel() > 0
              and weight.dtype in (torch.float32, torch.bfloat16) and torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if usable:
        if torch.is_grad_enabled() and weight.requires_grad:
            return _EmbeddingFn.apply(weight, ids, padding_idx)
        from ..layers import _bf16_weight
        from . import nn_kernels

        table = _bf16_weight(weight) if getattr(weight, "_bf16_shadow", None) is not None else weight.detach()
        return nn_kernels.embedding_fwd(table.contiguous(), ids)
    return F.embedding(ids, weight, padding_idx)


# ------------------------------------------------------------------------------ rotary embedding
class _RotaryQKFn(torch.autograd.Function):
    """Rotate q and k inside a fused qkv projection output, in place (the projection does not need its output for backward)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, seq, heads, head_dim, rot):
        from . import nn_kernels

        nn_kernels.rotary_qk_(qkv, cos, sin, seq, heads, head_dim, rot, 1.0)
        ctx.mark_dirty(qkv)
        ctx.save_for_backward(cos, sin)
        ctx.dims = (seq, heads, head_dim, rot)
        return qkv

    @staticmethod
    def backward(ctx, grad):
        from . import nn_kernels

        cos, sin = ctx.saved_tensors
        g = grad.contiguous()
        if g.data_ptr() == grad.data_ptr():
            g = grad.clone()
        nn_kernels.rotary_qk_(g, cos, sin, *ctx.dims, -1.0)
        return g, None, None, None, None, None, None


def rotary_qk_supported(qkv: torch.Tensor, head_dim: int, rot: int) -> bool:
    return _kernel_tensor(qkv) and qkv.is_contiguous() and rot % 16 == 0 and head_dim % 8 == 0 and rot > 0


def rotary_qk(qkv, cos_half, sin_half, seq: int, heads: int, head_dim: int, rot: int):
    """``qkv``: ``[B, S, heads * 3 * head_dim]`` bf16 (per-head interleaved q|k|v); tables ``[S, rot/2]`` fp32."""
    return _RotaryQKFn.apply(qkv, cos_half, sin_half, seq, heads, head_dim, rot)
