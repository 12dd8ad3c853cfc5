"""Surface selection, plan-then-mutate surgery, turbo schedule, step publishing."""

import pytest
import torch
from torch import nn

from stacr_b200 import STACRLinear, apply_stacr, select_target_names, set_step
from stacr_b200.compressor import STACRConfig
from stacr_b200.models import build_model
from stacr_b200.surgery import classify


def test_classify_uses_the_parent_block():
    assert classify("transformer.h.0.mlp.c_proj") == "mlp"
    assert classify("transformer.h.0.attn.c_proj") == "attention"
    assert classify("bert.encoder.layer.1.output.dense") == "mlp"
    assert classify("bert.encoder.layer.1.attention.output.dense") == "attention"
    assert classify("model.decoder.layers.3.fc1") == "mlp"
    assert classify("lm_head") is None


def test_surfaces_on_the_model_zoo():
    gpt = build_model("gpt-tiny")
    mlp = select_target_names(gpt, surface="mlp")
    assert len(mlp) == 8 and all(".mlp." in n for n in mlp)
    both = select_target_names(gpt, surface="mlp+attention")
    assert len(both) == 16
    neox = build_model("pythia-70m", num_hidden_layers=2, vocab_size=512)
    assert select_target_names(neox, surface="mlp") == [
        "gpt_neox.layers.0.mlp.dense_h_to_4h", "gpt_neox.layers.0.mlp.dense_4h_to_h",
        "gpt_neox.layers.1.mlp.dense_h_to_4h", "gpt_neox.layers.1.mlp.dense_4h_to_h",
    ]
    bert = build_model("bert-tiny")
    names = select_target_names(bert, surface="mlp", min_features=64)
    assert names == ["bert.encoder.layer.0.intermediate.dense", "bert.encoder.layer.0.output.dense",
                     "bert.encoder.layer.1.intermediate.dense", "bert.encoder.layer.1.output.dense"]


def test_apply_defaults_to_turbo_at_50_and_dataclass_none_means_full():
    model = build_model("gpt-tiny", n_layer=1)
    layers = apply_stacr(model)
    assert all(l.turbo_after_step == 50 for l in layers)
    assert STACRLinear.from_linear(nn.Linear(300, 8)).turbo_after_step is None
    model2 = build_model("gpt-tiny", n_layer=1)
    full = apply_stacr(model2, STACRConfig(min_features=128))
    assert all(l.turbo_after_step is None for l in full)


def test_turbo_switch_drops_residual_and_freezes_basis():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(300, 300), nn.GELU(), nn.Linear(300, 300))
    layers = apply_stacr(model, surface="all", turbo_after_step=2, residual_budget=0.01)
    x = torch.randn(16, 300)
    frozen = None
    for step in range(4):
        set_step(layers, step)
        out = model[0](x + step)
        n_saved = len(out.grad_fn.saved_tensors)
        assert n_saved == (6 if step < 2 else 3)
        if step == 2:
            frozen = layers[0].basis
        if step == 3:
            assert layers[0].basis is frozen


def test_invalid_option_leaves_model_untouched_and_unknown_keys_fail():
    model = build_model("gpt-tiny", n_layer=1)
    before = dict(model.named_modules())
    with pytest.raises(ValueError):
        apply_stacr(model, residual_bits=5)
    with pytest.raises(ValueError):
        apply_stacr(model, not_an_option=1)
    assert dict(model.named_modules()).keys() == before.keys()
    assert not any(isinstance(m, STACRLinear) for m in model.modules())
    with pytest.raises(ValueError):
        apply_stacr(model, surface="mlp", min_features=10**6)
    assert apply_stacr(model, surface="mlp", min_features=10**6, allow_empty=True) == []


def test_shared_module_is_wrapped_once_and_aliases_rebound():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(300, 300)
            self.b = self.a

    net = Net()
    layers = apply_stacr(net, surface="all")
    assert len(layers) == 1 and net.a is net.b is layers[0]
    assert layers[0].source_name == "a"


def test_parameter_identity_and_names_survive_surgery():
    model = build_model("gpt-tiny", n_layer=1)
    params = dict(model.named_parameters())
    apply_stacr(model)
    after = dict(model.named_parameters())
    assert after.keys() == params.keys()
    assert all(after[k] is params[k] for k in params)


def test_set_step_accepts_models_and_validates():
    model = build_model("gpt-tiny", n_layer=1)
    layers = apply_stacr(model)
    set_step(model, 7)
    assert all(l.step == 7 for l in layers)
    with pytest.raises(ValueError):
        set_step(layers, -1)
    with pytest.raises(ValueError):
        set_step(layers, 1, microbatch_index=2, accum_steps=2)
