"""Fidelity metrics (reference: stacr/metrics.py:6-55)."""

from __future__ import annotations

import torch


def cosine_similarity(
    reference: torch.Tensor,
    estimate: torch.Tensor,
    eps: float = 1e-12,
    *,
    reduction_dtype: torch.dtype = torch.float64,
) -> torch.Tensor:
    """Cosine of the flattened tensors; both zero -> 1, exactly one zero -> 0.

    Each vector is divided by its own max-magnitude before the reduction so that tiny or huge
    gradients neither underflow nor overflow.
    """
    if reference.shape != estimate.shape or reference.device != estimate.device:
        raise ValueError("Cosine inputs must have the same shape and device")
    if eps < 0 or reduction_dtype not in (torch.float32, torch.float64):
        raise ValueError("eps must be nonnegative; reduction_dtype must be float32 or float64")
    a = reference.detach().reshape(-1).to(reduction_dtype)
    b = estimate.detach().reshape(-1).to(reduction_dtype)
    if not (torch.isfinite(a).all() and torch.isfinite(b).all()):
        raise ValueError("Cosine inputs must be finite")
    if a.numel() == 0:
        return a.new_ones(())
    sa, sb = a.abs().amax(), b.abs().amax()
    if sa == 0 or sb == 0:
        return a.new_tensor(1.0 if (sa == 0 and sb == 0) else 0.0)
    a, b = a / sa, b / sb
    return (torch.dot(a, b) / (a.norm() * b.norm())).clamp(-1.0, 1.0)


def relative_mse(reference: torch.Tensor, estimate: torch.Tensor, eps: float = 1e-12) -> torch.Tensor:
    """Mean squared error divided by the mean reference energy."""
    r, e = reference.detach().float(), estimate.detach().float()
    return (r - e).square().mean() / r.square().mean().clamp_min(eps)


def gradient_cosine_from_activations(
    activation: torch.Tensor, reconstructed: torch.Tensor, grad_output: torch.Tensor
) -> torch.Tensor:
    """Cosine between ``G^T A`` and ``G^T A_hat`` for one linear layer."""
    flat = lambda t: t.reshape(-1, t.shape[-1]).float()
    g = flat(grad_output)
    return cosine_similarity(g.t() @ flat(activation), g.t() @ flat(reconstructed))
