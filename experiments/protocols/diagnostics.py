"""Measurement-only diagnostics of the protocol runner: activation reconstruction oracles and the boundary-codec drift tracker.

* Reconstruction oracles answer "how well would this layer's input be rebuilt from what the method keeps?" for one
  activation matrix: the compressed layer's own policy (current basis, coefficient and residual codecs, a *global* residual
  quota), a random-projection control, and a rank-matched truncated SVD of the same matrix.  They measure a policy, not the
  factors the backward pass actually used; the paired-gradient cosine is the runner's ``compute_grad_cosine``.
* ``C1DriftTracker`` watches the per-site residual energy of the checkpoint-boundary codecs next to the loss curve and
  records the first step at which a site's energy jumps while training is still finite ("finite drift"), and a slower
  worsening over a window.  The published negative result on boundary compression was diagnosed with this signal.

Behavioural parity: experiments/protocols/training.py:2155-2557 (drift) and :2745-2958 (oracles) of the reference project.
"""

from __future__ import annotations

import math
from collections import deque
from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn


# --------------------------------------------------------------------------------------------------------- oracles
def _flatten_last(t: torch.Tensor, features: int) -> torch.Tensor:
    return t.reshape(-1, features)


def _roundtrip_int(values: torch.Tensor, qmax: float, per_row: bool = False) -> torch.Tensor:
    if values.numel() == 0:
        return values
    amax = values.abs().amax(dim=1, keepdim=True) if per_row else values.abs().max()
    scale = (amax.float() / qmax).clamp_min(torch.finfo(torch.float32).tiny)
    return (torch.round(values.float() / scale).clamp_(-qmax, qmax) * scale).to(values.dtype)


def reconstruct_stacr_activation(module: nn.Module, activation_2d: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, Any]]:
    """Rebuild ``activation_2d`` the way the layer's current policy would: ``C Q^T`` plus the kept residual entries.

    Works for both engines.  Selection uses one global quota over the matrix (training uses per-chunk quotas for some
    modes); codecs follow the layer's configuration.  A layer without a usable basis returns the input itself.
    """
    basis = getattr(module, "effective_basis", None)
    if basis is None:
        basis = getattr(module, "basis", None)
    ready = bool(getattr(module, "basis_initialized", getattr(module, "_h_ready", None) or False))
    if hasattr(module, "basis_ready"):
        ready = ready or bool(module.basis_ready)
    if basis is None or basis.numel() == 0 or not ready:
        return activation_2d, {"reconstruction_scope": "baseline_or_uninitialized_basis", "rank": 0, "residual_mode": "baseline",
                               "residual_budget": 0.0, "residual_entries_kept": activation_2d.numel(), "coefficients_quantized": False,
                               "residuals_quantized": False}
    cfg = getattr(module, "config", None)
    state = getattr(module, "layer_state", {}) or {}
    rank = max(1, min(int(state.get("active_rank", basis.shape[1])), basis.shape[1]))
    q = basis[:, :rank].to(device=activation_2d.device, dtype=activation_2d.dtype)
    coeff = activation_2d @ q
    coeff_q = bool(getattr(cfg, "quantize_coefficients", False))
    coeff_used = _roundtrip_int(coeff, 127.0) if coeff_q else coeff
    low = coeff_used @ q.t()
    mode = str(getattr(cfg, "residual_mode", getattr(module, "residual_mode", "none")))
    budget = float(getattr(cfg, "residual_budget", getattr(module, "residual_budget", 0.0)))
    if hasattr(module, "_turbo") and module._turbo():
        mode, budget = "none", 0.0
    if cfg is not None and str(getattr(cfg, "post_warmup_residual_mode", "full")) == "none" and state.get("post_warmup", False):
        mode, budget = "none", 0.0
    residual = activation_2d - coeff @ q.t()
    kept = 0
    res_q = False
    total = residual.numel()
    k = int(round(budget * total))
    out = low
    if mode not in ("none", "baseline") and k > 0:
        flat = residual.reshape(-1)
        if mode == "block_sparse":
            bs = int(getattr(cfg, "residual_block_size", getattr(module, "residual_block_size", 16)))
            if residual.shape[1] % bs == 0:
                energy = residual.reshape(residual.shape[0], -1, bs).float().square().sum(-1).reshape(-1)
                blocks = energy.topk(max(1, k // bs)).indices
                idx = (blocks[:, None] * bs + torch.arange(bs, device=flat.device)).reshape(-1)
            else:
                idx = flat.abs().topk(min(k, total)).indices
        elif mode == "uniform":
            idx = torch.div(torch.arange(k, device=flat.device) * total, k, rounding_mode="floor")
        elif mode in ("threshold",):
            idx = (flat.abs() > float(getattr(cfg, "residual_threshold", 0.1))).nonzero(as_tuple=True)[0]
        else:   # topk, chunk_topk, global_topk, adaptive_threshold, sampled, sparse_only: the exact global top-k is their limit
            idx = flat.abs().topk(min(k, total)).indices
        vals = flat[idx]
        bits = int(getattr(cfg, "residual_quantize_bits", getattr(module, "residual_bits", 0)) or 0)
        if getattr(cfg, "quantize_residuals", bits in (4, 8)) and bits in (4, 8):
            vals = _roundtrip_int(vals, 7.0 if bits == 4 else 127.0)
            res_q = True
        sparse = torch.zeros_like(flat)
        sparse[idx] = vals
        out = low + sparse.view_as(residual)
        kept = int(idx.numel())
    return out, {"reconstruction_scope": "stacr_policy_global_quota", "rank": rank, "residual_mode": mode, "residual_budget": budget,
                 "residual_entries_kept": kept, "coefficients_quantized": coeff_q, "residuals_quantized": res_q}


def reconstruct_prac_activation(module: nn.Module, activation_2d: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, Any]]:
    """Random-projection control: ``(X P) P^T`` with the layer's fixed projection."""
    p = module.projection.to(device=activation_2d.device, dtype=activation_2d.dtype)
    return (activation_2d @ p) @ p.t(), {"reconstruction_scope": "prac_linear_random_projection", "rank": int(getattr(module, "effective_rank", p.shape[1])),
                                         "residual_mode": "none", "residual_budget": 0.0, "residual_entries_kept": 0, "coefficients_quantized": False,
                                         "residuals_quantized": False}


def reconstruct_svd_lowrank(activation_2d: torch.Tensor, rank: int, oversampling: int = 16, niter: int = 2) -> Tuple[torch.Tensor, Dict[str, Any]]:
    """Rank-matched truncated SVD of the same matrix (randomised, so wide GPT-2 inputs stay cheap): the per-batch optimum a
    tracked basis is compared with."""
    rows, feats = activation_2d.shape
    r = max(1, min(int(rank), rows, feats))
    width = min(max(r, r + max(0, int(oversampling))), rows, feats)
    work = activation_2d.float()
    try:
        u, s, v = torch.svd_lowrank(work, q=width, niter=max(0, int(niter)))
        recon, backend = (u[:, :r] * s[:r]) @ v[:, :r].t(), "torch.svd_lowrank"
    except RuntimeError:
        u, s, vh = torch.linalg.svd(work, full_matrices=False)
        recon, backend, width = (u[:, :r] * s[:r]) @ vh[:r], "torch.linalg.svd", r
    return recon.to(activation_2d.dtype), {"reconstruction_scope": "svd_lowrank_diagnostic_same_activation", "rank": r, "residual_mode": "none",
                                           "residual_budget": 0.0, "residual_entries_kept": 0, "coefficients_quantized": False,
                                           "residuals_quantized": False, "svd_backend": backend, "svd_q": int(width), "svd_niter": int(niter)}


def reconstruction_metrics(original: torch.Tensor, rebuilt: torch.Tensor) -> Dict[str, float]:
    a, b = original.reshape(-1).double(), rebuilt.reshape(-1).double()
    err = float((a - b).norm() / a.norm().clamp_min(1e-30))
    denom = float(a.norm() * b.norm())
    return {"relative_error": err, "cosine": float(torch.dot(a, b)) / denom if denom > 0 else 1.0}


@torch.no_grad()
def reconstruction_report(model: nn.Module, layers: List[nn.Module], run_forward, svd_rank: Optional[int] = None) -> Dict[str, Any]:
    """Capture every listed layer's input during ``run_forward()`` and report, per layer, how well each oracle rebuilds it."""
    captured: Dict[nn.Module, torch.Tensor] = {}
    handles = [layer.register_forward_pre_hook(lambda m, args: captured.__setitem__(m, args[0].detach())) for layer in layers]
    try:
        run_forward()
    finally:
        for h in handles:
            h.remove()
    names = {m: n for n, m in model.named_modules()}
    rows = []
    for layer in layers:
        x = captured.get(layer)
        if x is None:
            continue
        x2 = _flatten_last(x, x.shape[-1]).float()
        row: Dict[str, Any] = {"layer": names.get(layer, type(layer).__name__), "rows": int(x2.shape[0]), "features": int(x2.shape[1])}
        if hasattr(layer, "projection"):
            rec, info = reconstruct_prac_activation(layer, x2)
        else:
            rec, info = reconstruct_stacr_activation(layer, x2)
        row["method"] = {**info, **reconstruction_metrics(x2, rec)}
        rank = int(svd_rank or info.get("rank") or 8)
        srec, sinfo = reconstruct_svd_lowrank(x2, max(1, rank))
        row["svd"] = {**sinfo, **reconstruction_metrics(x2, srec)}
        rows.append(row)
    if not rows:
        return {"layers": [], "summary": None}
    mean = lambda key, field: sum(r[key][field] for r in rows) / len(rows)
    return {"layers": rows, "summary": {"method_relative_error_mean": mean("method", "relative_error"), "method_cosine_mean": mean("method", "cosine"),
                                        "svd_relative_error_mean": mean("svd", "relative_error"), "svd_cosine_mean": mean("svd", "cosine"), "count": len(rows)}}


# --------------------------------------------------------------------------------------------------------- C1 drift
def safe_perplexity(loss: float) -> Optional[float]:
    if loss is None or not math.isfinite(loss):
        return None
    return math.exp(min(float(loss), 50.0))


class C1DriftTracker:
    """First *finite* drift of the boundary codecs: a site's residual energy jumps while the loss is still finite.

    ``update`` is called once per optimizer step with the runtime's ``stats()`` (``per_site`` -> ``last_energy``,
    ``compressed_pack_count``) and the step's loss.  A *fast* event needs the leading site's energy to rise by at least
    ``energy_jump`` (absolute) and ``energy_ratio`` (relative) in one step together with a step perplexity above
    ``ppl_ratio`` times the best seen; a *slow* event needs the windowed mean perplexity to exceed the best windowed mean by
    ``slow_ratio``.  Only the first event of each kind is kept, with the site, the energies around it and the loss context.
    """

    def __init__(self, window: int = 20, energy_jump: float = 0.02, energy_ratio: float = 1.25, ppl_ratio: float = 1.15, slow_ratio: float = 1.10):
        self.window, self.energy_jump, self.energy_ratio, self.ppl_ratio, self.slow_ratio = window, energy_jump, energy_ratio, ppl_ratio, slow_ratio
        self.prev_energy: Dict[str, float] = {}
        self.losses: deque = deque(maxlen=window)
        self.step_ppl: deque = deque(maxlen=window)
        self.best_step_ppl: Optional[float] = None
        self.best_window_ppl: Optional[float] = None
        self.event: Optional[Dict[str, Any]] = None
        self.slow_event: Optional[Dict[str, Any]] = None
        self.first_nonfinite: Optional[Dict[str, Any]] = None
        self.memory_phase_peaks: Dict[str, int] = {}

    def note_memory(self, phase: str, allocated_bytes: int) -> None:
        self.memory_phase_peaks[phase] = max(int(allocated_bytes), self.memory_phase_peaks.get(phase, 0))

    def update(self, runtime_stats: Dict[str, Any], *, global_step: int, optimizer_step: int, loss_value: float) -> Dict[str, Any]:
        per_site = runtime_stats.get("per_site") or runtime_stats.get("sites") or {}
        current: Dict[str, float] = {}
        lead = None       # (delta, energy, site)
        for site, st in per_site.items():
            if int(st.get("compressed_pack_count", st.get("packs", 0)) or 0) <= 0:
                continue
            e = st.get("last_energy", st.get("last_residual_energy"))
            if not isinstance(e, (int, float)) or not math.isfinite(float(e)):
                continue
            e = float(e)
            current[str(site)] = e
            prev = self.prev_energy.get(str(site))
            delta = None if prev is None else e - prev
            key = (float("-inf") if delta is None else delta, e, str(site))
            if lead is None or key > lead:
                lead = key
            if self.first_nonfinite is None and st.get("first_nonfinite"):
                self.first_nonfinite = {"site": str(site), **dict(st["first_nonfinite"])}
        ppl = safe_perplexity(loss_value)
        finite = ppl is not None
        signal = None
        if finite:
            if self.best_step_ppl is not None and lead is not None and lead[0] != float("-inf"):
                site = lead[2]
                prev = self.prev_energy.get(site, 0.0)
                ratio = lead[1] / max(abs(prev), 1e-8)
                if lead[0] >= self.energy_jump and ratio >= self.energy_ratio and ppl >= self.ppl_ratio * self.best_step_ppl:
                    signal = "fast"
                    if self.event is None:
                        self.event = {"kind": "fast", "global_step": global_step, "optimizer_step": optimizer_step, "site": site, "energy": lead[1],
                                      "previous_energy": prev, "energy_delta": lead[0], "energy_ratio": ratio, "loss": loss_value, "step_perplexity": ppl,
                                      "best_step_perplexity": self.best_step_ppl}
            self.losses.append(float(loss_value))
            self.step_ppl.append(ppl)
            self.best_step_ppl = ppl if self.best_step_ppl is None else min(self.best_step_ppl, ppl)
            if len(self.step_ppl) == self.window:
                mean_ppl = sum(self.step_ppl) / self.window
                if self.best_window_ppl is not None and mean_ppl >= self.slow_ratio * self.best_window_ppl and self.slow_event is None:
                    self.slow_event = {"kind": "slow", "global_step": global_step, "optimizer_step": optimizer_step, "window_perplexity": mean_ppl,
                                       "best_window_perplexity": self.best_window_ppl, "leading_site": None if lead is None else lead[2]}
                    signal = signal or "slow"
                self.best_window_ppl = mean_ppl if self.best_window_ppl is None else min(self.best_window_ppl, mean_ppl)
        self.prev_energy = current
        return {"signal": signal, "leading_site": None if lead is None else lead[2], "leading_energy": None if lead is None else lead[1],
                "sites_tracked": len(current), "finite": finite}

    def summary(self) -> Dict[str, Any]:
        return {"first_finite_drift_event": self.event, "first_slow_drift_event": self.slow_event, "first_nonfinite_event": self.first_nonfinite,
                "best_step_perplexity": self.best_step_ppl, "memory_phase_peaks": dict(self.memory_phase_peaks)}
