"""Adaptive engine: exactness in every residual mode, state restore, replay, codecs, surgery."""

import copy

import pytest
import torch
from torch import nn

from stacr_b200.adaptive import (
    STACRConfig, STACRLinear, _choose_index_dtype, apply_adaptive_stacr, dequantize_int4, dequantize_int8, get_basis_pool,
    quantize_int4, quantize_int8, set_stacr_runtime_state,
)
from stacr_b200.adaptive_checkpointing import checkpoint


@pytest.mark.parametrize("mode", ["none", "topk", "threshold", "block_sparse", "adaptive_threshold", "sparse_only"])
def test_modes_keep_forward_and_input_gradient_exact(mode):
    torch.manual_seed(21)
    layer = STACRLinear(16, 7, STACRConfig(rank=4, residual_mode=mode, residual_budget=0.2))
    x = torch.randn(8, 16, requires_grad=True)
    r = x.detach().clone().requires_grad_(True)
    want = r.mm(layer.linear.weight.t()) + layer.linear.bias
    got = layer(x)
    assert torch.equal(got, want)
    g = torch.randn_like(got)
    got.backward(g)
    want.backward(g)
    assert torch.equal(x.grad, r.grad)
    assert torch.isfinite(layer.linear.weight.grad).all()


def test_state_dict_layout_and_controller_restore():
    cfg = STACRConfig(rank=4, residual_mode="topk", rank_mode="sensitivity", rank_min=1, rank_max=4, rank_adjust_interval=1,
                      freeze_basis_after_warmup=False, update_interval=1, lazy_update_enabled=False, oja_update_per_optimizer_step=True)
    first = STACRLinear(16, 7, cfg)
    set_stacr_runtime_state(first, 3)
    first(torch.randn(8, 16)).sum().backward()
    state = copy.deepcopy(first.state_dict())
    assert {"linear.weight", "linear.bias", "basis", "_basis_initialized", "step_counter", "_runtime_state"} <= set(state)
    assert state["_runtime_state"].dtype == torch.uint8
    second = STACRLinear(16, 7, copy.deepcopy(cfg))
    second.load_state_dict(state)
    assert second.layer_state == first.layer_state
    assert torch.equal(second.basis, first.basis) and second.basis_initialized
    for layer in (first, second):
        layer.zero_grad()
        set_stacr_runtime_state(layer, 4)
    x = torch.randn(8, 16)
    first(x).sum().backward()
    second(x).sum().backward()
    assert torch.equal(second.basis, first.basis)
    assert torch.equal(second.linear.weight.grad, first.linear.weight.grad)


def test_variance_rank_resizes_basis_and_reloads():
    cfg = STACRConfig(rank=8, rank_mode="variance", rank_min=1, rank_max=8, rank_variance_threshold=0.9)
    first = STACRLinear(16, 7, cfg)
    x = torch.randn(12, 1) @ torch.randn(1, 16)
    first(x).sum().backward()
    assert first.basis.shape[1] == 1
    second = STACRLinear(16, 7, copy.deepcopy(cfg))
    second.load_state_dict(first.state_dict())
    assert torch.equal(first.basis, second.basis) and second.basis_initialized


def test_saved_basis_survives_later_updates():
    layer = STACRLinear(16, 7, STACRConfig(rank=4, residual_mode="topk", freeze_basis_after_warmup=False, update_trigger="fixed",
                                           update_interval=2, lazy_update_enabled=False))
    x = torch.randn(8, 16)
    out = layer(x)
    held = out.grad_fn.basis.clone()
    layer(x * 2).sum().backward()
    assert torch.equal(out.grad_fn.basis, held)
    out.sum().backward()


@pytest.mark.parametrize("frozen", [False, True])
def test_checkpoint_guard_preserves_gradient(frozen):
    cfg = STACRConfig(rank=4, residual_mode="topk", residual_budget=0.2, freeze_basis_after_warmup=frozen, update_interval=1,
                      lazy_update_enabled=False)
    first = STACRLinear(16, 7, cfg)
    second = copy.deepcopy(first)
    x = torch.randn(8, 16, requires_grad=True)
    y = x.detach().clone().requires_grad_(True)
    first(x).square().sum().backward()
    checkpoint(second, y).square().sum().backward()
    assert torch.allclose(first.linear.weight.grad, second.linear.weight.grad)
    assert torch.equal(x.grad, y.grad)
    assert int(first.step_counter) == int(second.step_counter) == 1


@pytest.mark.parametrize("mode", ["eval", "no_grad", "frozen"])
def test_exact_paths_do_not_initialize(mode):
    layer = STACRLinear(16, 7, STACRConfig(rank=4))
    if mode == "eval":
        layer.eval()
    if mode == "frozen":
        layer.linear.weight.requires_grad_(False)
    with torch.set_grad_enabled(mode != "no_grad"):
        x = torch.randn(3, 16)
        assert torch.equal(layer(x), layer.linear(x))
    assert not layer.basis_initialized and int(layer.step_counter) == 0


def test_surgery_preserves_parameters_and_rng():
    model = nn.Sequential(nn.Linear(16, 7))
    params = list(model.parameters())
    rng = torch.get_rng_state()
    layers = apply_adaptive_stacr(model, {"rank": 4}, target_names=["0"])
    assert torch.equal(rng, torch.get_rng_state())
    assert all(a is b for a, b in zip(params, model.parameters()))
    assert layers[0].source_name == "0"
    model(torch.randn(8, 16)).sum().backward()
    with pytest.raises(ValueError):
        apply_adaptive_stacr(nn.Sequential(nn.Linear(16, 7)), rank=4, target_names=["0"], joint_qk=True)
    with pytest.raises(ValueError):
        apply_adaptive_stacr(nn.Sequential(nn.Linear(16, 7)), rank=4, target_names=["0"], bogus=1)


def test_conv1d_surgery_keeps_parameter_identity():
    class Conv1D(nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = nn.Parameter(torch.randn(16, 7))
            self.bias = nn.Parameter(torch.randn(7))

        def forward(self, x):
            return torch.addmm(self.bias, x, self.weight)

    model = nn.Sequential(Conv1D())
    weight = model[0].weight
    x = torch.randn(8, 16)
    want = model(x)
    apply_adaptive_stacr(model, rank=4, target_names=["0"])
    assert weight is model[0].linear.source_weight
    assert torch.allclose(model(x), want, atol=1e-5)
    model(x).sum().backward()
    assert weight.grad is not None and weight.grad.shape == weight.shape


@pytest.mark.parametrize("compression", ["csr", "delta"])
def test_index_compression_runs_backward(compression):
    layer = STACRLinear(16, 7, STACRConfig(rank=4, residual_mode="topk", residual_budget=0.3, index_compression=compression))
    layer(torch.randn(8, 16)).square().sum().backward()
    assert torch.isfinite(layer.linear.weight.grad).all()


@pytest.mark.parametrize("bits", [4, 8])
def test_factor_codecs_roundtrip(bits):
    x = torch.tensor([-2.0, -0.5, 0.0, 0.5, 2.0])
    if bits == 4:
        data, scale, length = quantize_int4(x)
        back = dequantize_int4(data, scale, length)
    else:
        data, scale = quantize_int8(x)
        back = dequantize_int8(data, scale)
    assert torch.all((back - x).abs() <= scale / 2 + 1e-6)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("value", [0.0, 6e-8])
def test_codecs_keep_zero_and_tiny_fp16_values(bits, value):
    v = torch.full((5,), value, dtype=torch.float16)
    if bits == 4:
        data, scale, length = quantize_int4(v)
        back = dequantize_int4(data, scale, length)
    else:
        data, scale = quantize_int8(v)
        back = dequantize_int8(data, scale)
    torch.testing.assert_close(back.float(), v.float(), rtol=0.01, atol=0)


def test_config_validation():
    for bad in (dict(streaming_algorithm="incremental_svd"), dict(update_interval=0), dict(residual_budget=2), dict(rank=0),
                dict(residual_quantize_bits=2), dict(basis_sharing="all", rank_mode="sensitivity"), dict(rank_min=9, rank_max=8)):
        with pytest.raises(ValueError):
            STACRConfig(**bad)
    assert _choose_index_dtype(100) == torch.int16
    assert _choose_index_dtype(2**20) == torch.int32
    assert _choose_index_dtype(2**32) == torch.int64


def test_basis_sharing_uses_one_pooled_basis():
    get_basis_pool().clear()
    model = nn.Sequential(nn.Linear(16, 16), nn.Linear(16, 16))
    layers = apply_adaptive_stacr(model, rank=4, basis_sharing="all", surface="all", min_features=1)
    model(torch.randn(8, 16)).sum().backward()
    assert layers[0]._resolve_basis() is layers[1]._resolve_basis()
    get_basis_pool().clear()


def test_turbofast_mapping_switches_to_low_rank_only():
    cfg = STACRConfig(rank=4, residual_mode="topk", residual_budget=0.2, post_warmup_residual_mode="none", residual_warmup_steps=2,
                      refresh_trigger="residual_energy", cache_basis_per_optimizer_step=True, oja_update_per_optimizer_step=True)
    layer = STACRLinear(16, 7, cfg)
    x = torch.randn(8, 16)
    names = []
    for step in range(4):
        set_stacr_runtime_state(layer, step)
        out = layer(x)
        names.append(type(out.grad_fn).__name__)
        out.sum().backward()
    assert "LowRankOnly" not in names[0] and "LowRankOnly" in names[3]
