"""Properties of the adaptive engine that follow from the method itself, checked on random shapes (hypothesis), independently of any
example-based expectation: what the compressed backward must reproduce exactly, what it may only approximate and by how much."""

import pytest
import torch
from hypothesis import given, settings, strategies as st

from stacr_b200.adaptive import STACRConfig, STACRLinear

MODES = ["none", "topk", "threshold", "block_sparse", "adaptive_threshold", "sparse_only"]
shapes = st.tuples(st.integers(4, 24), st.sampled_from([8, 16, 24, 32]), st.integers(1, 9))   # rows, in_features, out_features


def _layer_and_data(rows, feats, out, seed, **cfg):
    torch.manual_seed(seed)
    layer = STACRLinear(feats, out, STACRConfig(**cfg))
    x = torch.randn(rows, feats)
    g = torch.randn(rows, out)
    return layer, x, g


def _grads(layer, x, g):
    layer.linear.weight.grad = None
    layer.linear.bias.grad = None
    xin = x.clone().requires_grad_(True)
    layer(xin).backward(g)
    return xin.grad, layer.linear.weight.grad.clone(), layer.linear.bias.grad.clone()


@settings(max_examples=30, deadline=None, derandomize=True)
@given(shape=shapes, mode=st.sampled_from(MODES), seed=st.integers(0, 10 ** 6), rank=st.integers(1, 6))
def test_output_input_gradient_and_bias_gradient_do_not_depend_on_the_compression(shape, mode, seed, rank):
    rows, feats, out = shape
    layer, x, g = _layer_and_data(rows, feats, out, seed, rank=rank, residual_mode=mode, residual_budget=0.1)
    w, b = layer.linear.weight.detach(), layer.linear.bias.detach()
    assert torch.equal(layer(x), x @ w.t() + b)
    dx, _, db = _grads(layer, x, g)
    torch.testing.assert_close(dx, g @ w, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(db, g.sum(0), rtol=1e-5, atol=1e-6)


@settings(max_examples=20, deadline=None, derandomize=True)
@given(shape=shapes, seed=st.integers(0, 10 ** 6))
def test_weight_gradient_is_exact_when_nothing_is_discarded(shape, seed):
    """Either channel alone can carry everything: a basis of full width, or a residual budget of one."""
    rows, feats, out = shape
    dense = None
    for cfg in (dict(rank=feats, residual_mode="none"), dict(rank=1, residual_mode="topk", residual_budget=1.0, quantize_residuals=False),
                dict(rank=1, residual_mode="sparse_only", residual_budget=1.0, quantize_residuals=False)):
        layer, x, g = _layer_and_data(max(rows, feats), feats, out, seed, quantize_coefficients=False, **cfg)
        dense = g.t() @ x
        _, dw, _ = _grads(layer, x, g)
        torch.testing.assert_close(dw, dense, rtol=2e-3, atol=2e-3)


@settings(max_examples=25, deadline=None, derandomize=True)
@given(shape=shapes, seed=st.integers(0, 10 ** 6), rank=st.integers(1, 4), budget=st.sampled_from([0.0, 0.05, 0.3]))
def test_weight_gradient_error_obeys_the_bridge_bound(shape, seed, rank, budget):
    """``dW_c - dW = dY^T (X_hat - X)``, hence ``||dW_c - dW||_F <= ||dY||_2 ||X_hat - X||_F``.  ``||X_hat - X||_F`` is at most the
    distance of X to its best rank-r approximation *in the layer's current basis*, which the layer's own projector gives."""
    rows, feats, out = shape
    mode = "topk" if budget else "none"
    layer, x, g = _layer_and_data(rows, feats, out, seed, rank=rank, residual_mode=mode, residual_budget=budget or 0.005,
                                  quantize_coefficients=False, quantize_residuals=False)
    _, dw, _ = _grads(layer, x, g)           # the first call fixes the basis that was used for this very batch
    q = layer.basis.detach().float()[:, : layer.current_rank] if hasattr(layer, "current_rank") else layer.basis.detach().float()
    low_rank_error = (x - (x @ q) @ q.t()).norm()
    bound = torch.linalg.matrix_norm(g, ord=2) * low_rank_error
    assert (dw - g.t() @ x).norm() <= bound * (1 + 1e-4) + 1e-5


@settings(max_examples=15, deadline=None, derandomize=True)
@given(shape=shapes, seed=st.integers(0, 10 ** 6))
def test_more_residual_budget_never_hurts_the_weight_gradient_of_the_same_basis(shape, seed):
    rows, feats, out = shape
    errors = []
    for budget in (0.02, 0.2, 0.6):
        layer, x, g = _layer_and_data(rows, feats, out, seed, rank=2, residual_mode="topk", residual_budget=budget,
                                      quantize_coefficients=False, quantize_residuals=False)
        _, dw, _ = _grads(layer, x, g)
        # the error is dY^T E with E the unselected part of the residual; adding entries to the selection shrinks ||E||_F, and the
        # bound ||dY||_2 ||E||_F with it: compare through that bound, which is what the method guarantees
        q = layer.basis.detach().float()
        resid = x - (x @ q) @ q.t()
        k = max(1, int(round(budget * resid.numel())))
        kept = resid.abs().flatten().topk(min(k, resid.numel())).values
        errors.append(float((resid.norm() ** 2 - kept.square().sum()).clamp_min(0).sqrt()))
        assert (dw - g.t() @ x).norm() <= torch.linalg.matrix_norm(g, ord=2) * errors[-1] * (1 + 1e-3) + 1e-4
    assert errors[0] >= errors[1] >= errors[2]


def test_a_layer_in_eval_mode_or_without_grad_saves_nothing_compressed():
    layer, x, _ = _layer_and_data(8, 16, 4, 0, rank=2)
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t.shape) or t, lambda t: t):
        with torch.no_grad():
            layer(x)
    assert saved == []
