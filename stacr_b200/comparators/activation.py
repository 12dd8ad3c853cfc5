"""Basis controls that reuse the compressed layer's factor-native backward and change only how the basis is chosen.

``untracked`` = fixed random orthonormal basis, ``oasis`` = normalised Oja step from covariance eigenvectors,
``prac`` = half principal / half random directions refreshed on an interval, ``lowrank`` = tracked basis without a
residual.  Parity: comparators/activation.py:23-144 of the reference project.
"""

from __future__ import annotations

import inspect

import torch

from ..layers import STACRLinear
from ..oja import orthonormalize


def _fixed_randn(rows, cols, device, salt=0):
    gen = torch.Generator(device="cpu").manual_seed(1234 + rows + cols + salt)  # private generator: dropout stream untouched
    return torch.randn(rows, cols, generator=gen).to(device)


class _ComparatorBase(STACRLinear):
    """Shared bookkeeping: at most one basis change per step value."""

    def _claim_step(self) -> bool:
        self._sync_host()
        if self._h_ready and getattr(self, "_comparator_step", None) == self.step:
            return False
        self._comparator_step = self.step
        return True

    def _install(self, basis: torch.Tensor) -> None:
        self.basis = orthonormalize(basis.float()).to(self.basis.dtype)
        self._mark_updated(self.step)


class UntrackedLinear(_ComparatorBase):
    @torch.no_grad()
    def _refresh_basis(self, x2d):
        self._sync_host()
        if not self._h_ready:
            self._install(_fixed_randn(self.in_features, self.rank, x2d.device))


class OasisLinear(_ComparatorBase):
    gamma = 1.0

    @torch.no_grad()
    def _refresh_basis(self, x2d):
        if not self._claim_step():
            return
        x = x2d.detach().float()
        n = max(1, x.shape[0])
        if not self._h_ready:
            vectors = torch.linalg.eigh(x.t() @ x / n).eigenvectors
            self._install(vectors[:, -self.rank:])
            return
        q = self.basis.float()
        prod = x.t() @ (x @ q) / n
        scale = float(prod.norm()) / max(float(q.norm()), 1e-12)
        self._install(q + self.gamma / max(scale, 1e-12) * (prod - q @ (q.t() @ prod)))


class PracLinear(_ComparatorBase):
    principal_frac = 0.5
    refresh_every = 500

    @torch.no_grad()
    def _refresh_basis(self, x2d):
        if not self._claim_step():
            return
        if self._h_ready and self.step % int(self.refresh_every):
            return
        x = x2d.detach().float()
        k = min(self.rank, max(1, round(self.principal_frac * self.rank)), x.shape[0])
        basis = torch.linalg.svd(x, full_matrices=False).Vh[:k].t()
        if self.rank - k:
            basis = torch.cat([basis, _fixed_randn(self.in_features, self.rank - k, x.device, salt=2)], dim=1)
        self._install(basis)


class FatFunction(torch.autograd.Function):
    """Storage control: the same factors as the compressed layer, saved the wasteful way.

    ``basis_per_call`` saves a private copy of the basis with every call instead of a reference to the layer's one
    buffer; ``fat_residual`` saves int64 positions and fp32 values instead of narrow indices and quantised values.
    The arithmetic is the layer's reference arithmetic in PyTorch, so the only thing that moves between this control
    and the real layer is what autograd holds (parity: experiments/benchmarks/basis_storage.py:20-95).
    """

    @staticmethod
    def forward(ctx, x, weight, bias, basis, budget, residual_bits, chunk_rows, transposed, basis_per_call, fat_residual):
        from ..layers import _select_chunk_topk
        from ..quant import quantize_values

        feats = basis.shape[0]
        x2d = x.reshape(-1, feats)
        w = weight.to(x2d.dtype)
        out = x2d @ (w if transposed else w.t())
        if bias is not None:
            out = out + bias.to(out.dtype)
        q = basis.to(x2d.dtype)
        coeff = x2d @ q
        idx, val = _select_chunk_topk(x2d, coeff, q, float(budget), chunk_rows) if float(budget) > 0 else (None, None)
        saved = [coeff, weight, q.clone() if basis_per_call else basis]
        ctx.scale = None
        if idx is not None:
            if fat_residual or not residual_bits:
                saved += [idx.long() if fat_residual else idx, val.float() if fat_residual else val]
            else:
                packed = quantize_values(val, int(residual_bits))
                saved += [idx, packed.data]
                ctx.scale, ctx.bits, ctx.count = packed.scale, int(residual_bits), val.numel()
        ctx.save_for_backward(*saved)
        ctx.meta = (x.shape[:-1], feats, out.shape[1], bool(transposed), bias is not None and bias.requires_grad)
        return out.reshape(*x.shape[:-1], out.shape[1])

    @staticmethod
    def backward(ctx, dy):
        from ..quant import QuantizedValues

        lead, feats, outs, transposed, bias_grad = ctx.meta
        coeff, weight, q = ctx.saved_tensors[:3]
        g = dy.reshape(-1, outs)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            w = weight.to(g.dtype)
            dx = (g @ (w.t() if transposed else w)).reshape(*lead, feats)
        if ctx.needs_input_grad[1]:
            dw = (g.t() @ coeff.to(g.dtype)) @ q.to(g.dtype).t()
            if len(ctx.saved_tensors) > 3:
                idx, val = ctx.saved_tensors[3], ctx.saved_tensors[4]
                if ctx.scale is not None:
                    val = QuantizedValues(val, ctx.scale, ctx.bits, ctx.count).dequantize(torch.float32)
                rows, cols = torch.div(idx.long(), feats, rounding_mode="floor"), idx.long() % feats
                dw = dw.float().t().index_add(0, cols, g[rows].float() * val.float()[:, None]).t()
            dw = (dw.t() if transposed else dw).to(weight.dtype)
        if bias_grad:
            db = g.sum(0)
        return dx, dw, db, None, None, None, None, None, None, None


class FatLinear(STACRLinear):
    basis_per_call = True
    fat_residual = True

    def forward(self, x):
        if not (self.training and torch.is_grad_enabled() and self.weight.requires_grad) or x.numel() == 0:
            return self._exact(x)
        self._sync_host()
        self._refresh_basis(x.reshape(-1, self.in_features))
        budget = 0.0 if self._turbo() else self.residual_budget
        return FatFunction.apply(x, self.weight, self.bias, self.basis, budget, self.residual_bits, self.chunk_rows, self.transposed,
                                 self.basis_per_call, self.fat_residual)


def apply_fat(model, config: dict, basis_per_call: bool = True, fat_residual: bool = True):
    """Wrap the configured surface with the storage control; the two flags pick which saving is undone."""
    layers = apply_comparator(model, "fat", config)
    for layer in layers:
        layer.basis_per_call, layer.fat_residual = bool(basis_per_call), bool(fat_residual)
    return layers


COMPARATORS = {"fat": (FatLinear, 0.005), "stacr": (STACRLinear, 0.005), "lowrank": (STACRLinear, 0.0), "untracked": (UntrackedLinear, 0.0),
               "oasis": (OasisLinear, 0.0), "prac": (PracLinear, 0.0)}


def apply_comparator(model, kind: str, config: dict):
    """Replace the selected projections with the chosen basis control (Parameter identity and dtype preserved)."""
    from ..surgery import _is_conv1d, select_target_names

    if kind not in COMPARATORS:
        raise ValueError(f"Unknown basis comparator {kind!r}; choose {sorted(COMPARATORS)}")
    cls, budget = COMPARATORS[kind]
    cfg = dict(config)
    if kind in ("stacr", "fat"):
        cfg.setdefault("residual_budget", budget)
    else:
        cfg["residual_budget"] = 0.0
    names = select_target_names(model, surface=cfg.get("surface", "mlp"), min_features=cfg.get("min_features", 256), extra_names=cfg.get("extra_names", ()))
    accepted = set(inspect.signature(STACRLinear.__init__).parameters) - {"self", "weight", "bias", "transposed"}
    options = {k: v for k, v in cfg.items() if k in accepted}
    layers = []
    for name in names:
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        src = getattr(parent, leaf)
        layer = cls(src.weight, getattr(src, "bias", None), transposed=_is_conv1d(src), **options)
        layer.source_name = name
        layer.train(src.training)
        if isinstance(layer, PracLinear):
            layer.refresh_every, layer.principal_frac = int(cfg.get("refresh_every", 500)), float(cfg.get("principal_frac", 0.5))
        if isinstance(layer, FatLinear):
            layer.basis_per_call, layer.fat_residual = bool(cfg.get("basis_per_call", True)), bool(cfg.get("fat_residual", True))
        if isinstance(layer, OasisLinear):
            layer.gamma = float(cfg.get("gamma", 1.0))
        setattr(parent, leaf, layer)
        layers.append(layer)
    return layers
