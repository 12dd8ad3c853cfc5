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


COMPARATORS = {"stacr": (STACRLinear, 0.005), "lowrank": (STACRLinear, 0.0), "untracked": (UntrackedLinear, 0.0),
               "oasis": (OasisLinear, 0.0), "prac": (PracLinear, 0.0)}


def apply_comparator(model, kind: str, config: dict):
    """Replace the selected projections with the chosen basis control (Parameter identity and dtype preserved)."""
    from ..surgery import _is_conv1d, select_target_names

    if kind not in COMPARATORS:
        raise ValueError(f"Unknown basis comparator {kind!r}; choose {sorted(COMPARATORS)}")
    cls, budget = COMPARATORS[kind]
    cfg = dict(config)
    if kind == "stacr":
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
        if isinstance(layer, OasisLinear):
            layer.gamma = float(cfg.get("gamma", 1.0))
        setattr(parent, leaf, layer)
        layers.append(layer)
    return layers
