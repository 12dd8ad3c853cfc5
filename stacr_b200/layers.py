"""Projection-engine compressed linear layer.

``STACRLinear`` keeps a linear layer's forward output and input gradient exact and replaces
only what autograd saves for the weight gradient: rank-r coefficients ``C = X Q`` on a tracked
orthonormal basis ``Q`` plus a sparse, quantised residual ``S`` of ``X - C Q^T``.  Backward
contracts the factors directly, ``dW = (dY^T C) Q^T + dY^T S``; the dense input is never
rebuilt.  Behavioural parity target: stacr/layers.py:13-473 of the reference project
(constructor options, buffers and state_dict keys, selector semantics, saved-tensor
inventory, exact-path gate, checkpoint replay).

Two execution paths share this module:

* bf16 compute on a CUDA device runs the hand-written sm_100a kernels in
  ``stacr_b200.ops`` (tcgen05 GEMMs for the exact linear, the projection and the skinny
  ``A^T B`` products; radix-select residual selection; fused Oja + CholeskyQR2; bucketed sparse
  weight gradient).  There is no silent fallback: a missing kernel library raises.
* everything else (CPU, fp32/fp16) runs the PyTorch restatement below, which is also the
  numerical oracle the kernel tests compare against.
"""

from __future__ import annotations

import math
from typing import Any

import torch
from torch import nn
from torch.nn import functional as F

from .oja import oja_step, orthonormalize, seeded_random_basis, top_right_singular_basis
from .quant import QuantizedValues, quantize_values

RESIDUAL_MODES = {"chunk_topk", "topk", "global_topk", "uniform", "none", "block_sparse", "sampled"}

_BASIS_DTYPES = {
    "float32": torch.float32,
    "fp32": torch.float32,
    "float16": torch.float16,
    "fp16": torch.float16,
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
}


def _index_dtype(total: int) -> torch.dtype:
    return torch.int32 if total < 2**31 - 1 else torch.int64


def _chunk_bounds(rows: int, chunk_rows: int):
    step = max(1, int(chunk_rows))
    return [(lo, min(lo + step, rows)) for lo in range(0, rows, step)]


def _chunk_quota(budget: float, numel: int) -> int:
    return max(1, min(numel, int(round(budget * numel))))


# --------------------------------------------------------------------------------------
# Selector oracle (framework ops).  Each selector sees one chunk of the residual at a time so
# that the workspace stays chunk_rows x features.
# --------------------------------------------------------------------------------------
def _residual_chunk(x, coeff, basis, lo, hi):
    return (x[lo:hi] - coeff[lo:hi] @ basis.t()).reshape(-1)


def _select_chunk_topk(x, coeff, basis, budget, chunk_rows):
    rows, feats = x.shape
    k_total = int(round(float(budget) * rows * feats))
    if k_total <= 0:
        return None, None
    picked_i, picked_v = [], []
    for lo, hi in _chunk_bounds(rows, chunk_rows):
        e = _residual_chunk(x, coeff, basis, lo, hi)
        top = e.abs().topk(_chunk_quota(float(budget), e.numel()), sorted=False).indices
        picked_i.append(top + lo * feats)
        picked_v.append(e[top])
    idx, val = torch.cat(picked_i), torch.cat(picked_v)
    if idx.numel() > k_total:  # per-chunk rounding overshot the global budget: trim by magnitude
        keep = val.abs().topk(k_total, sorted=False).indices
        idx, val = idx[keep], val[keep]
    return idx.to(_index_dtype(rows * feats)), val


def _select_residual(x, coeff, basis, budget, chunk_rows, mode, block_size, sample_ratio):
    """Return ``(flat indices, values)`` of the stored residual entries, or ``(None, None)``."""
    if mode == "none" or budget <= 0 or x.numel() == 0:
        return None, None
    if mode in ("chunk_topk", "topk"):
        return _select_chunk_topk(x, coeff, basis, budget, chunk_rows)
    rows, feats = x.shape
    total = rows * feats
    k_total = int(round(budget * total))
    if k_total == 0:
        return None, None
    idt = _index_dtype(total)
    if mode == "block_sparse" and feats % block_size:
        return _select_chunk_topk(x, coeff, basis, budget, chunk_rows)
    if mode == "sampled":
        e = (x - coeff @ basis.t()).reshape(-1)
        mag = e.abs()
        gen = torch.Generator(device=x.device).manual_seed(0)
        probe = mag[torch.randint(total, (max(1024, int(total * sample_ratio)),), device=x.device, generator=gen)]
        cut = torch.quantile(probe.float(), 1.0 - budget)
        hits = (mag >= cut).nonzero(as_tuple=True)[0][:k_total]
        return hits.to(idt), e[hits]
    if mode == "global_topk":
        best_i = best_v = None
        for lo, hi in _chunk_bounds(rows, chunk_rows):
            e = _residual_chunk(x, coeff, basis, lo, hi)
            top = e.abs().topk(min(k_total, e.numel()), sorted=False).indices
            ci, cv = top + lo * feats, e[top]
            if best_i is not None:
                ci, cv = torch.cat((best_i, ci)), torch.cat((best_v, cv))
            keep = cv.abs().topk(min(k_total, cv.numel()), sorted=False).indices
            best_i, best_v = ci[keep], cv[keep]
        return best_i.to(idt), best_v
    out_i, out_v = [], []
    for lo, hi in _chunk_bounds(rows, chunk_rows):
        e = _residual_chunk(x, coeff, basis, lo, hi)
        if mode == "block_sparse":
            energy = e.reshape(-1, block_size).square().sum(1)
            count = max(1, int(round(budget * energy.numel())))
            blocks = energy.topk(count, sorted=False).indices
            local = (blocks[:, None] * block_size + torch.arange(block_size, device=x.device)).reshape(-1)
            out_i.append(local + lo * feats)
            out_v.append(e[local])
        elif mode == "uniform":
            first = math.ceil(lo * feats * k_total / total)
            last = math.ceil(hi * feats * k_total / total)
            absolute = torch.div(torch.arange(first, last, device=x.device) * total, k_total, rounding_mode="floor")
            out_i.append(absolute)
            out_v.append(e[absolute - lo * feats])
        else:
            raise ValueError(f"Unknown residual_mode: {mode!r}")
    return torch.cat(out_i).to(idt), torch.cat(out_v)


# --------------------------------------------------------------------------------------
# Kernel-path helpers
# --------------------------------------------------------------------------------------
# (old version, new version) of every basis rebound while a training step is being captured into a CUDA graph; None otherwise
GRAPH_BASIS_PAIRS: list | None = None


def _kernel_path(x: torch.Tensor, compute_dtype: torch.dtype) -> bool:
    return x.is_cuda and compute_dtype == torch.bfloat16


def _compute_dtype(x: torch.Tensor, weight: torch.Tensor) -> torch.dtype:
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type)
    return torch.promote_types(x.dtype, weight.dtype) if x.dtype != weight.dtype else x.dtype


def _bf16_weight(weight: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a master weight: the shadow the fused optimizer keeps current, else a cast.

    The shadow is trusted only while the master has not been written by anyone else.  The fused optimizer updates master
    and shadow through raw pointers (no version bump) and records the master's version counter next to the shadow; any
    other write (``load_state_dict``, a broadcast, another optimizer, a manual edit) bumps the counter, and the shadow is
    then refreshed from the master here before it is used.
    """
    shadow = getattr(weight, "_bf16_shadow", None)
    if shadow is not None and shadow.shape == weight.shape and shadow.device == weight.device:
        if getattr(weight, "_bf16_shadow_version", None) != weight._version:
            with torch.no_grad():
                shadow.copy_(weight.detach())
            weight._bf16_shadow_version = weight._version
        return shadow
    return weight.detach().to(torch.bfloat16)


def _basis_views(basis: torch.Tensor):
    """bf16 ``[N, r]`` copy and padded transpose of one basis *version*, cached on the tensor object.

    A basis version is never mutated (updates rebind the buffer), so object identity is a valid key.
    """
    cached = getattr(basis, "_sb_views", None)
    if cached is None:
        from .ops import stacr_ops

        qb = basis.detach().to(torch.bfloat16).contiguous()
        cached = (qb, stacr_ops.pad_basis_transpose(qb))
        basis._sb_views = cached
    return cached


_ZERO_FACTORS: dict = {}


def _zero_factors(rows: int, cols: int, device):
    """Cached all-zero rank-1 coefficient column ``[rows, 1]`` and basis ``[cols, 1]`` (bf16)."""
    key = (rows, cols, device)
    hit = _ZERO_FACTORS.get(key)
    if hit is None:
        if len(_ZERO_FACTORS) > 64:
            _ZERO_FACTORS.clear()
        hit = (torch.zeros(rows, 1, dtype=torch.bfloat16, device=device), torch.zeros(cols, 1, dtype=torch.bfloat16, device=device))
        _ZERO_FACTORS[key] = hit
    return hit


def _select_residual_kernels(x, coeff, qb, budget, chunk_rows, mode, block_size, sample_ratio, bits):
    """Kernel-path selection.  Returns ``(idx, QuantizedValues)`` or ``(None, None)``."""
    from .ops import stacr_ops

    if mode == "none" or budget <= 0 or x.numel() == 0:
        return None, None
    rows, feats = x.shape
    total = rows * feats
    k_total = int(round(float(budget) * total))
    if k_total <= 0:
        return None, None
    idt = _index_dtype(total)
    if mode == "block_sparse" and feats % block_size:
        mode = "chunk_topk"
    if mode in ("chunk_topk", "topk", "global_topk"):
        if mode == "global_topk":
            quotas, chunk = [min(k_total, total)], rows
        else:
            chunk = max(1, int(chunk_rows))
            quotas = [_chunk_quota(float(budget), (hi - lo) * feats) for lo, hi in _chunk_bounds(rows, chunk)]
        over = sum(quotas) - k_total
        if over > 0 and mode != "global_topk":
            # the per-chunk roundings overshoot the global budget: select unquantised, trim the
            # few smallest entries, then quantise what is kept
            idx, val, _ = stacr_ops.residual_topk(x, coeff, qb, quotas, chunk, 0, idt)
            keep = val.float().abs().topk(k_total, sorted=False).indices
            return idx[keep], quantize_values(val[keep], bits)
        idx, val, scale = stacr_ops.residual_topk(x, coeff, qb, quotas, chunk, bits, idt)
        if bits == 4:
            from .quant import pack_int4

            val = pack_int4(val)
        return idx, QuantizedValues(val, scale, bits, int(idx.numel()))
    if mode == "uniform":
        idx = torch.div(torch.arange(k_total, device=x.device) * total, k_total, rounding_mode="floor").to(idt)
        return idx, quantize_values(stacr_ops.residual_gather(x, coeff, qb, idx), bits)
    if mode == "block_sparse" and block_size % 8 == 0 and block_size <= 256 and not (block_size & (block_size - 1)):
        energy = stacr_ops.residual_block_energy(x, coeff, qb, block_size)  # [rows, feats/bs]
        per_row = feats // block_size
        bounds = list(_chunk_bounds(rows, chunk_rows))
        counts = [max(1, int(round(budget * (hi - lo) * per_row))) for lo, hi in bounds]
        if per_row % 8 == 0 and len(bounds) <= 16 and rows * per_row < 2 ** 31:
            # the radix-select kernel run on the block energies themselves: with a zero rank-1 basis its "residual" is its input,
            # so one call ranks every chunk's blocks (by bf16-rounded energy, the resolution every selector here uses)
            zc, zq = _zero_factors(rows, per_row, x.device)
            blocks, _, _ = stacr_ops.residual_topk(energy.to(torch.bfloat16), zc, zq, counts, max(1, int(chunk_rows)), 0, torch.int32)
            blocks = blocks.long()
        else:
            blocks = torch.cat([energy[lo:hi].reshape(-1).topk(c, sorted=False).indices + lo * per_row for (lo, hi), c in zip(bounds, counts)])
        idx = (blocks[:, None] * block_size + torch.arange(block_size, device=x.device)).reshape(-1).to(idt)
        return idx, quantize_values(stacr_ops.residual_gather(x, coeff, qb, idx), bits)
    if mode == "sampled" and feats % 8 == 0:
        # the same selector without the dense residual: the probe is a gather of residual values at the random positions, the cut
        # is the probe's quantile, and one pass over X lists the entries at or above the cut; the first k_total of them in index
        # order are kept, as in the framework form (the cut is lowered by one bf16 step so that ">=" survives the strict compare)
        gen = torch.Generator(device=x.device).manual_seed(0)
        pos = torch.randint(total, (max(1024, int(total * sample_ratio)),), device=x.device, generator=gen)
        probe = stacr_ops.residual_gather(x, coeff, qb, pos).float().abs()
        cut = float(torch.quantile(probe, 1.0 - float(budget)))
        idx, val = stacr_ops.residual_above(x, coeff, qb, cut * (1.0 - 2.0 ** -8) if cut > 0 else -1.0)
        keep = val.float().abs() >= cut
        idx, val = idx[keep], val[keep]
        if idx.numel() == 0:
            return None, None
        order = torch.argsort(idx)[:k_total]
        return idx[order].to(idt), quantize_values(val[order], bits)
    # odd block sizes (and sampled on widths that are no multiple of 8): framework ops
    idx, val = _select_residual(x, coeff, qb, budget, chunk_rows, mode, block_size, sample_ratio)
    if idx is None:
        return None, None
    return idx, quantize_values(val, bits)


class STACRFunction(torch.autograd.Function):
    """Exact forward / input gradient; factor-native weight gradient.

    Saved for backward: ``coeff, weight, q`` and, with a residual, ``idx, qdata, qscale`` -- never
    a tensor the size of the input.  The basis passed in is an immutable version.
    """

    @staticmethod
    def forward(
        ctx,
        x,
        weight,
        bias,
        basis,
        budget,
        residual_bits,
        chunk_rows,
        transposed,
        residual_mode="chunk_topk",
        residual_block_size=16,
        residual_sample_ratio=0.1,
        tp=None,
    ):
        # ``tp``: a ``parallel.tp.TPContext`` when this layer is a tensor-parallel shard.  A row-parallel shard sums its
        # output over the ranks inside the forward GEMM; a column-parallel shard sums its input gradient inside the backward GEMM.
        feats = basis.shape[0]
        x2d = x.reshape(-1, feats)
        cdt = _compute_dtype(x, weight)
        ctx.kernel_path = _kernel_path(x2d, cdt)
        if ctx.kernel_path:
            from .ops import stacr_ops
            from .ops.gemm import gemm

            xa = x2d.to(torch.bfloat16).contiguous()
            wb = _bf16_weight(weight)
            bf = None if bias is None else bias.detach().float()
            # Conv1D keeps W as [in, out]: that is the MN-major B operand of the same kernel
            if tp is not None and tp.kind == "row":
                out2d = tp.gemm_sum(xa, wb.contiguous(), b_mn=bool(transposed), bias=bf)
            else:
                out2d = gemm(xa, wb, b_mn=bool(transposed), bias=bf)
            qb, qt = _basis_views(basis)
            coeff = stacr_ops.project(xa, qt)[:, : basis.shape[1]].to(torch.bfloat16)
            idx, packed = _select_residual_kernels(
                xa, coeff, qb, float(budget), int(chunk_rows), residual_mode, int(residual_block_size),
                float(residual_sample_ratio), int(residual_bits),
            )
            q = qb
        else:
            if transposed:
                out2d = x2d.mm(weight) if bias is None else torch.addmm(bias, x2d, weight)
            else:
                out2d = F.linear(x2d, weight, bias)
            if tp is not None and tp.kind == "row":
                out2d = tp.sum_(out2d)
            # compression arithmetic runs in the linear's output dtype with ambient autocast off
            with torch.autocast(device_type=x.device.type, enabled=False):
                act, q = x2d.to(out2d.dtype), basis.to(out2d.dtype)
                coeff = act.mm(q)
                idx, val = _select_residual(
                    act, coeff, q, float(budget), int(chunk_rows), residual_mode, int(residual_block_size),
                    float(residual_sample_ratio),
                )
                packed = quantize_values(val, int(residual_bits)) if val is not None else None
        tensors = [coeff, weight, q]
        if idx is not None:
            tensors += [idx, packed.data, packed.scale]
        ctx.save_for_backward(*tensors)
        ctx.has_residual = idx is not None
        ctx.residual_bits = packed.bits if packed is not None else 0
        ctx.residual_len = packed.length if packed is not None else 0
        ctx.leading, ctx.in_features = x.shape[:-1], feats
        ctx.out_features, ctx.transposed = out2d.shape[1], bool(transposed)
        ctx.input_dtype = x.dtype
        ctx.bias_dtype = None if bias is None else bias.dtype
        ctx.n_args = len(ctx.needs_input_grad)
        ctx.tp = tp
        return out2d.reshape(*ctx.leading, ctx.out_features)

    @staticmethod
    def backward(ctx, grad_out):
        coeff, weight, q, *res = ctx.saved_tensors
        g2d = grad_out.reshape(-1, ctx.out_features)
        gx = gw = gb = None
        if ctx.kernel_path:
            from .ops import stacr_ops
            from .ops.gemm import gemm

            ga = g2d.to(torch.bfloat16).contiguous()
            if ctx.needs_input_grad[0]:
                wb = _bf16_weight(weight)
                # dX = dY W: W[out, in] is MN-major for this product; Conv1D's [in, out] is K-major
                if ctx.tp is not None and ctx.tp.kind == "column":
                    gx = ctx.tp.gemm_sum(ga, wb.contiguous(), b_mn=not ctx.transposed)
                else:
                    gx = gemm(ga, wb, b_mn=not ctx.transposed)
                gx = gx.reshape(*ctx.leading, ctx.in_features).to(ctx.input_dtype)
            if ctx.needs_input_grad[1]:
                residual = None
                if ctx.has_residual and res[0].numel():
                    residual = (res[0], res[1], res[2], ctx.residual_bits, ctx.residual_len)
                sink = getattr(weight, "_sb_grad_sink", None)
                if sink is not None and weight.dtype == torch.float32:
                    # the kernel delivers dW into the flat gradient buffer (and across ranks) itself
                    stacr_ops.weight_grad(ga, coeff, q.float(), residual, ctx.out_features, ctx.in_features, ctx.transposed, torch.float32, sink=sink)
                    sink.done()
                else:
                    # a gradient synchroniser may lend the parameter's slot of its flat buffer for the first
                    # backward pass after zero_grad: the kernel then writes there and nothing is copied or accumulated
                    slot = getattr(weight, "_sb_grad_out", None) if getattr(weight, "_sb_grad_fresh", False) else None
                    if slot is not None and slot.dtype == weight.dtype:
                        weight._sb_grad_fresh = False
                    else:
                        slot = None
                    gw = stacr_ops.weight_grad(
                        ga, coeff, q.float(), residual, ctx.out_features, ctx.in_features, ctx.transposed, weight.dtype
                        if weight.dtype in (torch.float32, torch.bfloat16) else torch.float32, out=slot,
                    ).to(weight.dtype)
                    ready = getattr(weight, "_sb_grad_ready", None) if slot is not None else None
                    if ready is not None and not getattr(weight, "_sb_tied", False):
                        ready()          # the slot is the gradient: nothing goes back through autograd (it would be cloned)
                        gw = None
            if ctx.needs_input_grad[2]:
                from .ops.nn_ops import bias_grad

                gb = bias_grad(ga).to(ctx.bias_dtype)
            return (gx, gw, gb) + (None,) * (ctx.n_args - 3)
        with torch.autocast(device_type=g2d.device.type, enabled=False):
            if ctx.needs_input_grad[0]:
                w = weight.to(g2d.dtype)
                gx = g2d.mm(w.t() if ctx.transposed else w)
                if ctx.tp is not None and ctx.tp.kind == "column":
                    gx = ctx.tp.sum_(gx)
                gx = gx.reshape(*ctx.leading, ctx.in_features).to(ctx.input_dtype)
            if ctx.needs_input_grad[1]:
                gw = (g2d.t() @ coeff.to(g2d.dtype)) @ q.to(g2d.dtype).t()
                if ctx.has_residual and res[0].numel():
                    idx, qdata, qscale = res
                    wide = torch.float64 if g2d.dtype == torch.float64 else torch.float32
                    vals = QuantizedValues(qdata, qscale, ctx.residual_bits, ctx.residual_len).dequantize(wide)
                    flat = idx.long()
                    r_i = torch.div(flat, ctx.in_features, rounding_mode="floor")
                    c_i = flat - r_i * ctx.in_features
                    # S^T dY accumulated per stored entry (duplicates add up, as a coalesced COO would)
                    corr = torch.zeros(ctx.in_features, ctx.out_features, dtype=wide, device=g2d.device)
                    gwide = g2d.to(wide)
                    for lo in range(0, flat.numel(), 1 << 15):  # bounded gather workspace
                        sl = slice(lo, lo + (1 << 15))
                        corr.index_add_(0, c_i[sl], gwide[r_i[sl]] * vals[sl, None])
                    gw = gw + corr.t().to(gw.dtype)
                if ctx.transposed:
                    gw = gw.t()
                gw = gw.to(weight.dtype)
            if ctx.needs_input_grad[2]:
                gb = g2d.sum(0).to(ctx.bias_dtype)
        return (gx, gw, gb) + (None,) * (ctx.n_args - 3)


def _check_positive_int(name: str, value) -> None:
    if isinstance(value, bool) or int(value) != value or value < 1:
        raise ValueError(f"{name} must be a positive integer")


def _check_optional_step(name: str, value) -> None:
    if value is not None and (isinstance(value, bool) or int(value) != value or value < 0):
        raise ValueError(f"{name} must be a nonnegative integer")


class STACRLinear(nn.Module):
    """Linear projection whose saved input is compressed; parameters are the original objects.

    Call :func:`stacr_b200.set_step` (or ``layer.set_step``) with the optimizer step before each
    training forward.  All forwards of one step share one basis version (gradient accumulation,
    checkpoint replay).  Eval mode, ``no_grad`` and frozen weights take the plain linear path and
    leave the basis untouched.  After ``turbo_after_step`` the basis freezes and no residual is
    stored; the weights keep training.
    """

    def __init__(
        self,
        weight: nn.Parameter,
        bias: nn.Parameter | None,
        *,
        rank: int = 8,
        residual_budget: float = 0.005,
        residual_bits: int = 8,
        oja_lr: float = 0.01,
        update_interval: int = 1,
        warmup_steps: int = 0,
        freeze_after_warmup: bool = False,
        turbo_after_step: int | None = None,
        chunk_rows: int = 512,
        basis_dtype: str = "float32",
        transposed: bool = False,
        residual_mode: str = "chunk_topk",
        residual_block_size: int = 16,
        residual_sample_ratio: float = 0.1,
    ):
        super().__init__()
        if not isinstance(weight, nn.Parameter) or weight.ndim != 2 or not weight.is_floating_point():
            raise ValueError("weight must be a floating-point 2-D Parameter")
        _check_positive_int("rank", rank)
        _check_positive_int("update_interval", update_interval)
        _check_positive_int("chunk_rows", chunk_rows)
        _check_positive_int("residual_block_size", residual_block_size)
        if not math.isfinite(residual_budget) or not 0 <= residual_budget <= 1:
            raise ValueError("residual_budget must be between 0 and 1")
        if residual_bits not in (0, 4, 8):
            raise ValueError("residual_bits must be 0, 4, or 8")
        if not math.isfinite(oja_lr) or oja_lr < 0:
            raise ValueError("oja_lr must be finite and nonnegative")
        _check_optional_step("warmup_steps", warmup_steps)
        _check_optional_step("turbo_after_step", turbo_after_step)
        if residual_mode not in RESIDUAL_MODES:
            raise ValueError(f"residual_mode must be one of {sorted(RESIDUAL_MODES)}")
        if not math.isfinite(residual_sample_ratio) or not 0 < residual_sample_ratio <= 1:
            raise ValueError("residual_sample_ratio must be in (0, 1]")
        if basis_dtype in ("auto", "activation"):
            store_dtype = weight.dtype
        elif basis_dtype in _BASIS_DTYPES:
            store_dtype = _BASIS_DTYPES[basis_dtype]
        else:
            raise ValueError(f"Unknown basis_dtype: {basis_dtype!r}")
        self.weight, self.bias = weight, bias
        self.transposed = bool(transposed)
        in_dim, out_dim = (0, 1) if self.transposed else (1, 0)
        self.in_features, self.out_features = int(weight.shape[in_dim]), int(weight.shape[out_dim])
        if bias is not None and (bias.ndim != 1 or bias.numel() != self.out_features):
            raise ValueError("bias shape must match the output feature count")
        self.rank = min(int(rank), self.in_features)
        self.residual_budget = float(residual_budget)
        self.residual_bits = int(residual_bits)
        self.oja_lr = float(oja_lr)
        self.update_interval = int(update_interval)
        self.warmup_steps = int(warmup_steps)
        self.freeze_after_warmup = bool(freeze_after_warmup)
        self.turbo_after_step = turbo_after_step
        self.chunk_rows = int(chunk_rows)
        self.residual_mode = residual_mode
        self.residual_block_size = int(residual_block_size)
        self.residual_sample_ratio = float(residual_sample_ratio)
        dev = weight.device
        self.register_buffer("basis", torch.zeros(self.in_features, self.rank, dtype=store_dtype, device=dev))
        self.register_buffer("basis_ready", torch.zeros((), dtype=torch.bool, device=dev))
        self.register_buffer("_step", torch.zeros((), dtype=torch.int64, device=dev))
        self.register_buffer("_last_update_step", torch.full((), -1, dtype=torch.int64, device=dev))
        # Host mirrors of the three scalar buffers: schedules are decided on the host without a
        # device->host read per layer per forward.  ``None`` means "re-read the buffer".
        self._h_step: int | None = 0
        self._h_last: int | None = -1
        self._h_ready: bool | None = False

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_linear(cls, module: nn.Module, **options) -> "STACRLinear":
        """Wrap an ``nn.Linear`` or a Transformers ``Conv1D`` (weight stored as ``[in, out]``)."""
        conv1d = type(module).__name__ == "Conv1D"
        if not (isinstance(module, nn.Linear) or conv1d):
            raise TypeError("from_linear requires nn.Linear or Transformers Conv1D")
        layer = cls(module.weight, getattr(module, "bias", None), transposed=conv1d, **options)
        layer.train(module.training)
        return layer

    # ------------------------------------------------------------------ scalar state
    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self._h_step = self._h_last = self._h_ready = None

    def _sync_host(self) -> None:
        if self._h_step is None:
            self._h_step = int(self._step.item())
            self._h_last = int(self._last_update_step.item())
            self._h_ready = bool(self.basis_ready.item())

    @property
    def step(self) -> int:
        self._sync_host()
        return self._h_step

    @step.setter
    def step(self, value: int) -> None:
        self.set_step(value)

    def set_step(self, step: int) -> None:
        if isinstance(step, bool) or int(step) != step or step < 0:
            raise ValueError("step must be a nonnegative integer")
        self._sync_host()
        if int(step) != self._h_step:
            self._h_step = int(step)
            self._step.fill_(int(step))

    def _mark_updated(self, step: int, ready: bool = True) -> None:
        self._h_last = step
        self._last_update_step.fill_(step)
        if ready and not self._h_ready:
            self._h_ready = True
            self.basis_ready.fill_(True)

    def _turbo(self) -> bool:
        return self.turbo_after_step is not None and self.step >= int(self.turbo_after_step)

    # ------------------------------------------------------------------ basis maintenance
    def _initial_basis(self, x2d: torch.Tensor) -> torch.Tensor:
        if x2d.shape[0] < self.rank:
            return seeded_random_basis(self.in_features, self.rank, x2d.device, seed=0)
        if x2d.is_cuda and x2d.dtype == torch.bfloat16:
            from .ops.basis import range_finder_basis

            return range_finder_basis(x2d, self.rank)
        return top_right_singular_basis(x2d.detach(), self.rank)

    @torch.no_grad()
    def _refresh_basis(self, x2d: torch.Tensor) -> None:
        if not x2d.numel():
            return
        step = self.step
        if self._h_ready and self._h_last == step:
            return
        store = self.basis.dtype
        with torch.autocast(device_type=x2d.device.type, enabled=False):
            if not self._h_ready:
                # rebind: a graph that saved the previous tensor keeps its version
                self.basis = self._initial_basis(x2d).to(store)
                self._mark_updated(step)
                return
            if self.freeze_after_warmup and step >= self.warmup_steps:
                return
            if self._turbo() or step % self.update_interval:
                return
            if x2d.is_cuda and x2d.dtype == torch.bfloat16:
                from .ops.basis import oja_step_kernels

                previous = self.basis
                self.basis = oja_step_kernels(previous, x2d, self.oja_lr).to(store)
                if GRAPH_BASIS_PAIRS is not None:
                    # the step is being captured into a CUDA graph: replays read the basis from `previous`'s storage, so the
                    # capture ends by copying the new version back there (see graphs.GraphedStep)
                    GRAPH_BASIS_PAIRS.append((previous, self.basis))
            else:
                self.basis = oja_step(self.basis, x2d.detach(), self.oja_lr).to(store)
            self._mark_updated(step, ready=False)

    # ------------------------------------------------------------------ forward
    def _exact(self, x: torch.Tensor) -> torch.Tensor:
        tp = getattr(self, "tp_context", None)
        if tp is not None:
            return tp.exact(x, self)
        if not self.transposed:
            return F.linear(x, self.weight, self.bias)
        flat = x.reshape(-1, self.in_features)
        y = flat.mm(self.weight) if self.bias is None else torch.addmm(self.bias, flat, self.weight)
        return y.reshape(*x.shape[:-1], self.out_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.ndim < 1 or x.shape[-1] != self.in_features:
            raise ValueError(f"Expected last input dimension {self.in_features}, got {tuple(x.shape)}")
        if not (self.training and torch.is_grad_enabled() and self.weight.requires_grad) or x.numel() == 0:
            return self._exact(x)
        from .adaptive_checkpointing import get_global_recomputation_guard

        guard = get_global_recomputation_guard()
        replayed = guard.replay_layer(self) if guard.is_recomputing else None
        if replayed is not None:
            basis, budget = replayed
        else:
            self._sync_host()
            if not guard.is_recomputing or not self._h_ready:
                x2d = x.reshape(-1, self.in_features)
                if x2d.is_cuda and _compute_dtype(x, self.weight) == torch.bfloat16:
                    x2d = x2d.to(torch.bfloat16)
                self._refresh_basis(x2d)
            basis = self.basis
            budget = 0.0 if self._turbo() else self.residual_budget
            guard.record_layer(self, (basis, budget))
        return STACRFunction.apply(
            x, self.weight, self.bias, basis, budget, self.residual_bits, self.chunk_rows, self.transposed,
            self.residual_mode, self.residual_block_size, self.residual_sample_ratio, getattr(self, "tp_context", None),
        )

    # ------------------------------------------------------------------ accounting
    def _residual_count(self, rows: int, budget: float) -> int:
        n = self.in_features
        count = int(round(budget * rows * n))
        if not count:
            return 0
        spans = [hi - lo for lo, hi in _chunk_bounds(rows, self.chunk_rows)]
        if self.residual_mode == "block_sparse" and n % self.residual_block_size == 0:
            bs = self.residual_block_size
            return sum(max(1, int(round(budget * span * n / bs))) * bs for span in spans)
        if self.residual_mode in ("chunk_topk", "topk", "block_sparse"):
            return min(count, sum(max(1, int(round(budget * span * n))) for span in spans))
        return count

    def stored_bytes(self, rows: int, value_bytes: int = 2) -> dict[str, Any]:
        """Bytes one forward keeps for backward (factors only; no weights, no workspaces).

        Chunk and block quotas include their rounding; ``sampled`` reports an upper bound because
        its count depends on the data.  ``basis`` is the persistent buffer plus the per-forward
        cast when its width differs from ``value_bytes``.
        """
        if isinstance(rows, bool) or int(rows) != rows or rows < 0 or value_bytes not in (2, 4, 8):
            raise ValueError("rows must be a nonnegative integer and value_bytes must be 2, 4, or 8")
        rows = int(rows)
        budget = 0.0 if (self._turbo() or self.residual_mode == "none") else self.residual_budget
        count = self._residual_count(rows, budget)
        idx_bytes = 4 if rows * self.in_features < 2**31 - 1 else 8
        if self.residual_bits == 4:
            val_bytes = (count + 1) // 2
        else:
            val_bytes = count * (1 if self.residual_bits == 8 else value_bytes)
        coeff = rows * self.rank * value_bytes
        residual = count * idx_bytes + val_bytes + (4 if count else 0)
        persistent = self.basis.numel() * self.basis.element_size()
        cast = self.basis.numel() * value_bytes if (self.basis.element_size() != value_bytes and rows) else 0
        return {
            "coeff": coeff,
            "residual": residual,
            "basis": persistent + cast,
            "total": coeff + residual + persistent + cast,
            "persistent_basis": persistent,
            "saved_basis_cast": cast,
            "residual_count": count,
            "residual_count_is_upper_bound": self.residual_mode == "sampled",
        }
