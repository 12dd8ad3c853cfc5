"""Gradient low-rank-projection optimizers, in-tree (no external packages).

``GaLoreAdamW``: for each selected 2-D parameter the gradient is projected onto a rank-r subspace found by an SVD of
the gradient every ``update_proj_gap`` steps; Adam moments live in the projected space (``r x n`` instead of
``m x n``) and the update is projected back and scaled.  ``SubTrackAdamW``: the same projected-moment scheme, but the
subspace is *tracked* between refreshes with a Grassmannian step along the gradient's out-of-subspace component
instead of being recomputed, and the moments are rotated with the basis.  These stand in for the external
optimizers the reference adapts (comparators/galore_adapter.py, comparators/subtrack_adapter.py there).
"""

from __future__ import annotations

import torch


class GaLoreAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @staticmethod
    def _projector(grad: torch.Tensor, rank: int, proj_type: str):
        g = grad.float()
        left = g.shape[0] >= g.shape[1] if proj_type == "std" else proj_type == "left"
        if proj_type in ("reverse_std",):
            left = g.shape[0] < g.shape[1]
        u, _, vh = torch.linalg.svd(g, full_matrices=False)
        r = min(rank, *g.shape)
        return ("right", vh[:r].t().contiguous()) if left else ("left", u[:, :r].contiguous())

    def _track(self, st, grad, group):
        """Hook for subclasses: adjust ``st['proj']`` between refreshes."""

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                g = p.grad
                lowrank = "rank" in group and p.dim() == 2
                if lowrank:
                    if "proj" not in st or (st["step"] - 1) % int(group.get("update_proj_gap", 200)) == 0:
                        st["side"], st["proj"] = self._projector(g, int(group["rank"]), group.get("proj_type", "std"))
                        st.pop("exp_avg", None)
                    else:
                        self._track(st, g, group)
                    proj = st["proj"].to(g.dtype)
                    g_low = g @ proj if st["side"] == "right" else proj.t() @ g
                else:
                    g_low = g
                if "exp_avg" not in st or st["exp_avg"].shape != g_low.shape:
                    st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(g_low, dtype=torch.float32), torch.zeros_like(g_low, dtype=torch.float32)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(g_low.float(), alpha=1 - b1)
                v.mul_(b2).addcmul_(g_low.float(), g_low.float(), value=1 - b2)
                upd = (m / (1 - b1 ** st["step"])) / ((v / (1 - b2 ** st["step"])).sqrt() + group["eps"])
                if lowrank:
                    proj = st["proj"].float()
                    upd = (upd @ proj.t() if st["side"] == "right" else proj @ upd) * float(group.get("scale", 0.25))
                p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(upd.to(p.dtype), alpha=-group["lr"])
        return loss

    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for st in self.state.values() for t in st.values() if torch.is_tensor(t))


class SubTrackAdamW(GaLoreAdamW):
    def _track(self, st, grad, group):
        every = int(group.get("track_interval", 10))
        if st["step"] % every:
            return
        q = st["proj"].float()
        g = grad.float()
        a = g if st["side"] == "left" else g.t()        # columns live in the space q spans
        low = q.t() @ a
        resid = a - q @ low                             # out-of-subspace part of the gradient
        tangent = resid @ low.t()                       # Grassmannian direction that reduces the projection error
        norm = tangent.norm()
        if norm > 0:
            new_q = torch.linalg.qr(q + float(group.get("step_size", 0.1)) * tangent / norm).Q
            rot = new_q.t() @ q                          # carry the moments into the new coordinates
            if "exp_avg" in st:
                if st["side"] == "left":
                    st["exp_avg"] = rot @ st["exp_avg"]
                    st["exp_avg_sq"] = (rot.abs() @ st["exp_avg_sq"])
                else:
                    st["exp_avg"] = st["exp_avg"] @ rot.t()
                    st["exp_avg_sq"] = st["exp_avg_sq"] @ rot.abs().t()
            st["proj"] = new_q.contiguous()


def split_param_groups(model, target_modules, weight_decay, **lowrank_kwargs):
    low, rest = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        hit = p.dim() == 2 and (any(t in name for t in target_modules) if target_modules else True)
        (low if hit else rest).append(p)
    groups = []
    if rest:
        groups.append({"params": rest, "weight_decay": weight_decay})
    if low:
        groups.append({"params": low, "weight_decay": weight_decay, **lowrank_kwargs})
    if not groups:
        raise ValueError("No parameters to optimize")
    return groups
