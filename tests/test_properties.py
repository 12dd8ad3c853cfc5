"""Properties of the projection engine and its codecs on random inputs (hypothesis), stated from the method rather than from
examples: round trips, error bounds of the quantisers, selector budgets and the optimality of the exact selectors."""

import math

import pytest
import torch
from hypothesis import given, settings, strategies as st
from torch import nn

from stacr_b200.index_compression import compress_indices, decompress_indices
from stacr_b200.layers import STACRFunction
from stacr_b200.quant import QuantizedValues, pack_int4, quantize_values, unpack_int4


@settings(max_examples=60, deadline=None, derandomize=True)
@given(rows=st.integers(1, 40), cols=st.integers(1, 300), frac=st.floats(0.0, 1.0), mode=st.sampled_from(["none", "csr", "delta"]),
       keep_order=st.booleans(), wide=st.booleans(), seed=st.integers(0, 10 ** 6))
def test_index_codecs_are_lossless_for_any_subset(rows, cols, frac, mode, keep_order, wide, seed):
    g = torch.Generator().manual_seed(seed)
    total = rows * cols
    k = int(frac * total)
    chosen = torch.randperm(total, generator=g)[:k].to(torch.int64 if wide else torch.int32)
    packed = compress_indices(chosen, rows, cols, mode, preserve_order=keep_order)
    back = decompress_indices(packed)
    assert back.dtype == chosen.dtype and back.numel() == k
    if keep_order or mode == "none":
        assert torch.equal(back, chosen)
    else:
        assert torch.equal(back.sort().values, chosen.sort().values)
    if k:
        assert packed.memory_bytes() > 0


@settings(max_examples=60, deadline=None, derandomize=True)
@given(n=st.integers(1, 500), bits=st.sampled_from([4, 8]), scale=st.floats(1e-6, 1e4), seed=st.integers(0, 10 ** 6))
def test_quantiser_error_is_at_most_half_a_step_of_the_largest_value(n, bits, scale, seed):
    g = torch.Generator().manual_seed(seed)
    values = torch.randn(n, generator=g) * scale
    q = quantize_values(values, bits)
    back = q.dequantize(torch.float32)
    levels = 2 ** (bits - 1) - 1
    step = float(values.abs().max()) / levels
    assert back.shape == values.shape
    assert float((back - values).abs().max()) <= 0.5 * step * (1 + 1e-4) + 1e-12
    assert torch.equal(quantize_values(torch.zeros(n), bits).dequantize(torch.float32), torch.zeros(n))


@settings(max_examples=40, deadline=None, derandomize=True)
@given(n=st.integers(0, 257), seed=st.integers(0, 10 ** 6))
def test_int4_packing_round_trips_every_length(n, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-7, 8, (n,), generator=g, dtype=torch.int8)
    packed = pack_int4(codes)
    assert packed.numel() == (n + 1) // 2
    assert torch.equal(unpack_int4(packed, n), codes)


def _saved_selection(x, q, budget, mode, chunk_rows=16, block=8, bits=0):
    w = nn.Parameter(torch.zeros(3, x.shape[1], dtype=x.dtype))
    y = STACRFunction.apply(x, w, None, q, budget, bits, chunk_rows, False, mode, block, 0.5)
    saved = y.grad_fn.saved_tensors
    coeff, _, qs = saved[:3]
    if len(saved) == 3:
        return coeff, qs, torch.empty(0, dtype=torch.long), torch.empty(0, dtype=x.dtype)
    idx, data, scale = saved[3:]
    return coeff, qs, idx.long(), QuantizedValues(data, scale, bits, idx.numel()).dequantize(x.dtype)


@settings(max_examples=40, deadline=None, derandomize=True)
@given(rows=st.integers(2, 40), feats=st.sampled_from([8, 16, 40]), rank=st.integers(1, 4), budget=st.floats(0.01, 0.5), seed=st.integers(0, 10 ** 6))
def test_global_topk_keeps_exactly_the_budget_and_nothing_larger_is_left_out(rows, feats, rank, budget, seed):
    torch.manual_seed(seed)
    x = torch.randn(rows, feats, dtype=torch.float64)
    q = torch.linalg.qr(torch.randn(feats, rank, dtype=torch.float64)).Q
    coeff, qs, idx, vals = _saved_selection(x, q, budget, "global_topk")
    residual = (x - coeff @ qs.t()).flatten()
    k = int(round(budget * rows * feats))
    assert idx.numel() == k and idx.unique().numel() == k
    if k:
        torch.testing.assert_close(vals, residual[idx])
        left = residual.abs().clone()
        left[idx] = 0
        assert float(left.max()) <= float(vals.abs().min()) + 1e-12


@settings(max_examples=40, deadline=None, derandomize=True)
@given(rows=st.integers(2, 48), feats=st.sampled_from([8, 16, 40]), budget=st.floats(0.02, 0.4), chunk=st.sampled_from([4, 16, 64]),
       mode=st.sampled_from(["chunk_topk", "uniform", "block_sparse", "sampled"]), seed=st.integers(0, 10 ** 6))
def test_every_selector_stores_true_residual_values_at_distinct_positions_within_budget(rows, feats, budget, chunk, mode, seed):
    torch.manual_seed(seed)
    x = torch.randn(rows, feats, dtype=torch.float64)
    q = torch.linalg.qr(torch.randn(feats, 2, dtype=torch.float64)).Q
    coeff, qs, idx, vals = _saved_selection(x, q, budget, mode, chunk_rows=chunk)
    residual = (x - coeff @ qs.t()).flatten()
    assert idx.unique().numel() == idx.numel() and (idx.numel() == 0 or int(idx.max()) < rows * feats)
    if idx.numel():
        torch.testing.assert_close(vals, residual[idx])
    total = rows * feats
    # chunk and block quotas round per chunk (at least one entry or block each): allow that slack on top of the budget
    n_chunks = math.ceil(rows / chunk)
    slack = n_chunks * (8 if mode == "block_sparse" else 1) + 8
    assert idx.numel() <= budget * total + slack


@settings(max_examples=30, deadline=None, derandomize=True)
@given(rows=st.integers(4, 32), feats=st.sampled_from([8, 24]), out=st.integers(1, 6), bits=st.sampled_from([0, 4, 8]),
       mode=st.sampled_from(["chunk_topk", "global_topk", "none"]), seed=st.integers(0, 10 ** 6))
def test_weight_gradient_error_is_bounded_by_what_was_discarded(rows, feats, out, bits, mode, seed):
    """``dW_c - dW = dY^T (X_hat - X)`` with ``X_hat`` the stored reconstruction, so the Frobenius error is at most
    ``||dY||_2 ||X_hat - X||_F``; forward output and input gradient stay exact."""
    torch.manual_seed(seed)
    x = torch.randn(rows, feats, dtype=torch.float64, requires_grad=True)
    w = nn.Parameter(torch.randn(out, feats, dtype=torch.float64))
    q = torch.linalg.qr(torch.randn(feats, 3, dtype=torch.float64)).Q
    y = STACRFunction.apply(x, w, None, q, 0.1, bits, 8, False, mode, 8, 0.5)
    assert torch.equal(y, x.detach() @ w.detach().t())
    saved = y.grad_fn.saved_tensors
    coeff, _, qs = saved[:3]
    x_hat = coeff @ qs.t()
    if len(saved) > 3:
        idx, data, scale = saved[3:]
        x_hat = x_hat.flatten().index_add(0, idx.long(), QuantizedValues(data, scale, bits, idx.numel()).dequantize(torch.float64)).view(rows, feats)
    g = torch.randn(rows, out, dtype=torch.float64)
    y.backward(g)
    torch.testing.assert_close(x.grad, g @ w.detach())
    err = (w.grad - g.t() @ x.detach()).norm()
    assert float(err) <= float(torch.linalg.matrix_norm(g, ord=2) * (x_hat - x.detach()).norm()) * (1 + 1e-9) + 1e-12
