"""Mechanism diagnostics: the activation-error -> gradient-error inequality, residual gain, byte ledger.

Parity: stacr/analysis.py:12-114 of the reference project.
"""

from __future__ import annotations

import math

import torch

from .metrics import cosine_similarity


def _safe_ratio(num: float, den: float):
    return num / den if den else None


def _cos_from_error(eps):
    return math.sqrt(max(0.0, 1 - eps * eps)) if eps is not None and eps < 1 else None


@torch.no_grad()
def gradient_bridge(activation: torch.Tensor, reconstruction: torch.Tensor, grad_output: torch.Tensor, *, spectral: bool = True) -> dict:
    """Check ``|G^T (A - A_hat)| <= |G| |A - A_hat|`` and the cosine bounds that follow from it.

    ``spectral=True`` uses the 2-norm of the upstream gradient, ``False`` the cheaper Frobenius
    norm (a weaker bound).  Relative quantities are ``None`` when the exact gradient is zero.
    """
    if activation.shape != reconstruction.shape or activation.ndim < 2:
        raise ValueError("Activation and reconstruction must have the same matrix-like shape")
    a = activation.detach().reshape(-1, activation.shape[-1]).double()
    a_hat = reconstruction.detach().reshape_as(a).double()
    g = grad_output.detach().reshape(-1, grad_output.shape[-1]).double()
    if a.shape[0] != g.shape[0] or len({a.device, a_hat.device, g.device}) != 1:
        raise ValueError("Activations and upstream gradients must share row count and device")
    if not all(bool(torch.isfinite(t).all()) for t in (a, a_hat, g)):
        raise ValueError("Diagnostic inputs must be finite")
    err = a - a_hat
    exact, approx, delta = g.t() @ a, g.t() @ a_hat, g.t() @ err
    norm = lambda t: float(torch.linalg.vector_norm(t))
    n_a, n_err, n_exact, n_delta = norm(a), norm(err), norm(exact), norm(delta)
    n_g = float(torch.linalg.matrix_norm(g, ord=2 if spectral else "fro"))
    eps = _safe_ratio(n_delta, n_exact)
    upper = _safe_ratio(n_g * n_err, n_exact)
    cos = float(cosine_similarity(exact, approx))
    sharp = _cos_from_error(eps)
    return {
        "activation_relative_error": _safe_ratio(n_err, n_a),
        "gradient_relative_error": eps,
        "cosine": cos,
        "gradient_error_upper": upper,
        "kappa": _safe_ratio(n_g * n_a, n_exact),
        "sharp_cosine_bound": sharp,
        "activation_cosine_bound": _cos_from_error(upper),
        "bridge_holds": n_delta <= n_g * n_err + 1e-10 * max(1, n_exact),
        "cosine_bound_holds": (cos + 1e-10 >= sharp) if sharp is not None else None,
        "cosine_error_proxy": (1 - cos) / (1 + cos) if cos > -1 else None,
        "upstream_norm": "spectral" if spectral else "frobenius",
    }


def residual_proxy_gain(cosine_on: float, cosine_off: float) -> float | None:
    """``1 - (e_on / e_off)^2`` with ``e = (1 - c) / (1 + c)``: the cosine-based residual gain."""
    for c in (cosine_on, cosine_off):
        if not (math.isfinite(c) and -1 < c <= 1):
            raise ValueError("Cosines must be finite and in (-1, 1]")
    e_on = (1 - cosine_on) / (1 + cosine_on)
    e_off = (1 - cosine_off) / (1 + cosine_off)
    return 1 - (e_on / e_off) ** 2 if e_off else None


def surface_ledger(wrapped_bytes: int, payload_bytes: int, baseline_peak_bytes: int, *, basis_bytes: int = 0,
                   workspace_bytes: int | None = None) -> dict:
    """Saved-surface predictor plus separately measured persistent (basis) and workspace costs."""
    from .memory import saved_surface_predictor

    if min(wrapped_bytes, payload_bytes, basis_bytes) < 0 or (workspace_bytes is not None and workspace_bytes < 0):
        raise ValueError("Byte counts must be nonnegative")
    saving = wrapped_bytes - payload_bytes
    return {
        "wrapped_bytes": wrapped_bytes,
        "payload_bytes": payload_bytes,
        "activation_saving_bytes": saving,
        "ssp": saved_surface_predictor(saving, baseline_peak_bytes),
        "basis_bytes": basis_bytes,
        "workspace_bytes": workspace_bytes,
        "net_after_basis_bytes": saving - basis_bytes,
        "net_after_workspace_bytes": None if workspace_bytes is None else saving - basis_bytes - workspace_bytes,
    }
