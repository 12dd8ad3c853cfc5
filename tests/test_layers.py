"""Projection-engine layer: exactness, saved-tensor inventory, basis versioning, resume, replay."""

import copy

import pytest
import torch
from torch import nn

import stacr_b200 as S
from stacr_b200.adaptive_checkpointing import checkpoint
from stacr_b200.layers import STACRFunction, STACRLinear, _select_residual
from stacr_b200.quant import QuantizedValues


def _pair(in_f=32, out_f=12, **opts):
    torch.manual_seed(0)
    lin = nn.Linear(in_f, out_f)
    ref = copy.deepcopy(lin)
    return STACRLinear.from_linear(lin, **opts), lin, ref


def test_forward_and_input_gradient_are_bit_exact():
    layer, lin, ref = _pair(rank=4, residual_budget=0.05)
    x = torch.randn(20, 32, requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    y, yr = layer(x), ref(xr)
    assert torch.equal(y, yr)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert torch.equal(x.grad, xr.grad)
    assert torch.equal(lin.bias.grad, ref.bias.grad)


def test_no_saved_tensor_is_as_large_as_the_input_and_inventory_counts():
    layer, lin, _ = _pair(in_f=64, rank=4, residual_budget=0.02)
    x = torch.randn(128, 64)
    y = layer(x)
    saved = y.grad_fn.saved_tensors
    assert len(saved) == 6
    assert all(t.numel() < x.numel() for t in saved if t is not lin.weight)
    layer.turbo_after_step = 3
    layer.set_step(3)
    assert len(layer(x).grad_fn.saved_tensors) == 3


def test_basis_is_rebound_never_mutated():
    layer, _, _ = _pair(rank=4)
    x = torch.randn(16, 32)
    layer.set_step(0)
    first = layer(x)
    held = first.grad_fn.saved_tensors[2]
    snapshot = held.clone()
    version = held._version
    layer.set_step(1)
    layer(x * 2).sum().backward()
    assert held._version == version and torch.equal(held, snapshot)
    first.sum().backward()


def test_state_dict_keys_and_resume_reproduces_basis_and_gradients():
    layer, lin, _ = _pair(rank=4, residual_budget=0.05)
    x = torch.randn(24, 32)
    for step in range(3):
        layer.set_step(step)
        layer(x + step).sum().backward()
    keys = set(layer.state_dict())
    assert keys == {"weight", "bias", "basis", "basis_ready", "_step", "_last_update_step"}
    clone, lin2, _ = _pair(rank=4, residual_budget=0.05)
    clone.load_state_dict(copy.deepcopy(layer.state_dict()))
    assert clone.step == 2 and torch.equal(clone.basis, layer.basis)
    for l, p in ((layer, lin), (clone, lin2)):
        p.weight.grad = None
        l.set_step(3)
        l(x).sum().backward()
    assert torch.equal(layer.basis, clone.basis)
    assert torch.equal(lin.weight.grad, lin2.weight.grad)


@pytest.mark.parametrize("mode", ["eval", "no_grad", "frozen", "empty"])
def test_exact_paths_have_no_basis_side_effects(mode):
    layer, lin, ref = _pair(rank=4)
    if mode == "eval":
        layer.eval()
    if mode == "frozen":
        lin.weight.requires_grad_(False)
    x = torch.randn(0 if mode == "empty" else 5, 32)
    with torch.set_grad_enabled(mode != "no_grad"):
        assert torch.equal(layer(x), ref(x))
    assert not bool(layer.basis_ready) and int(layer._last_update_step) == -1


def test_checkpoint_replay_matches_direct_gradient():
    a, lin_a, _ = _pair(rank=4, residual_budget=0.1)
    b = copy.deepcopy(a)
    x = torch.randn(16, 32, requires_grad=True)
    z = x.detach().clone().requires_grad_(True)
    a(x).square().sum().backward()
    checkpoint(b, z).square().sum().backward()
    assert torch.allclose(lin_a.weight.grad, b.weight.grad)
    assert torch.equal(x.grad, z.grad)
    assert torch.equal(a.basis, b.basis)


@pytest.mark.parametrize("mode", ["chunk_topk", "topk", "global_topk", "uniform", "block_sparse", "sampled"])
@pytest.mark.parametrize("bits", [0, 4, 8])
def test_weight_gradient_is_the_factor_identity(mode, bits):
    torch.manual_seed(5)
    rows, n, o, r = 40, 32, 9, 4
    x = torch.randn(rows, n, dtype=torch.float64)
    w = nn.Parameter(torch.randn(o, n, dtype=torch.float64))
    q = torch.linalg.qr(torch.randn(n, r, dtype=torch.float64)).Q
    y = STACRFunction.apply(x, w, None, q, 0.1, bits, 16, False, mode, 8, 0.5)
    coeff, _, qs, idx, data, scale = y.grad_fn.saved_tensors
    vals = QuantizedValues(data, scale, bits, idx.numel()).dequantize(torch.float64)
    sparse = torch.zeros(rows * n, dtype=torch.float64)
    sparse.index_add_(0, idx.long(), vals)
    g = torch.randn(rows, o, dtype=torch.float64)
    y.backward(g)
    expected = g.t() @ (coeff @ qs.t() + sparse.view(rows, n))
    torch.testing.assert_close(w.grad, expected)


def test_global_topk_is_exact_regardless_of_chunking():
    torch.manual_seed(7)
    x = torch.randn(37, 24)
    q = torch.linalg.qr(torch.randn(24, 3)).Q
    c = x @ q
    e = (x - c @ q.t()).reshape(-1)
    k = int(round(0.1 * e.numel()))
    want = set(e.abs().topk(k).indices.tolist())
    for chunk in (1, 5, 16, 64):
        idx, val = _select_residual(x, c, q, 0.1, chunk, "global_topk", 16, 0.1)
        assert set(idx.tolist()) == want
        torch.testing.assert_close(val, e[idx.long()])


def test_conv1d_weights_are_handled_transposed():
    class Conv1D(nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = nn.Parameter(torch.randn(32, 12))
            self.bias = nn.Parameter(torch.randn(12))

        def forward(self, x):
            return torch.addmm(self.bias, x, self.weight)

    torch.manual_seed(1)
    conv = Conv1D()
    layer = STACRLinear.from_linear(conv, rank=4, residual_budget=0.1)
    assert layer.transposed and (layer.in_features, layer.out_features) == (32, 12)
    x = torch.randn(10, 32, requires_grad=True)
    y = layer(x)
    assert torch.equal(y, conv(x))
    y.sum().backward()
    assert conv.weight.grad.shape == conv.weight.shape


@pytest.mark.parametrize("mode", ["chunk_topk", "global_topk", "block_sparse", "uniform", "none"])
@pytest.mark.parametrize("bits", [0, 4, 8])
def test_stored_bytes_equals_saved_inventory(mode, bits):
    layer, lin, _ = _pair(in_f=64, rank=4, residual_budget=0.03, residual_mode=mode, residual_bits=bits, chunk_rows=16,
                          basis_dtype="float32")
    x = torch.randn(50, 64)
    y = layer(x)
    saved = [t for t in y.grad_fn.saved_tensors if t is not lin.weight]
    actual = sum(t.numel() * t.element_size() for t in saved)
    report = layer.stored_bytes(50, value_bytes=4)
    # the saved q is the persistent basis itself when dtypes match
    assert report["total"] - report["saved_basis_cast"] == actual


def test_invalid_options_raise():
    lin = nn.Linear(8, 4)
    for bad in (dict(rank=0), dict(residual_budget=1.5), dict(residual_bits=3), dict(residual_mode="nope"), dict(chunk_rows=0),
                dict(basis_dtype="int8"), dict(turbo_after_step=-1), dict(oja_lr=float("nan")), dict(residual_sample_ratio=0)):
        with pytest.raises(ValueError):
            STACRLinear.from_linear(lin, **bad)
    with pytest.raises(TypeError):
        STACRLinear.from_linear(nn.ReLU())
    assert S.STACRLinear is STACRLinear
