"""Memory baselines, optional-package adapters, diagnostics context, transfer and graph protocols, CLI exit codes."""

import json
import os
import subprocess
import sys

import pytest
import torch
from torch import nn

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ------------------------------------------------------------------------------------------------ baselines
def test_amp_manager_modes():
    from stacr_b200.protocols.baselines.amp import AMPManager, resolve_amp_dtype

    assert resolve_amp_dtype("none", "cpu") == (None, False)
    assert resolve_amp_dtype("bf16", "cpu")[0] == torch.bfloat16
    amp = AMPManager("bf16", "cpu")
    lin = nn.Linear(8, 8)
    opt = torch.optim.SGD(lin.parameters(), lr=0.1)
    before = lin.weight.detach().clone()
    with amp.autocast():
        out = lin(torch.randn(4, 8))
        assert out.dtype == torch.bfloat16
    amp.backward(out.float().square().mean())
    amp.unscale_(opt)
    amp.step(opt)
    assert not torch.equal(lin.weight, before) and amp.get_scale() == 1.0
    assert AMPManager("none", "cpu").enabled is False
    assert amp.state_dict()["amp_mode"] == "bf16"
    with pytest.raises(ValueError):
        resolve_amp_dtype("fp8", "cpu")


def test_saved_tensor_offload_and_factor_compressor_roundtrip():
    from stacr_b200.protocols.baselines.offload import OffloadManager, SavedTensorOffloader
    from stacr_b200.protocols.baselines.saved_tensor_compressor import SavedTensorCompressor

    off = SavedTensorOffloader("cpu", min_bytes=64)
    w = nn.Parameter(torch.randn(64, 64))
    x = torch.randn(32, 64, requires_grad=True)
    with off.context():
        y = (x @ w).relu().sum()
    y.backward()
    ref_x = torch.autograd.grad((x @ w).relu().sum(), x)[0]
    torch.testing.assert_close(x.grad, ref_x)
    stats = off.get_timing_stats()
    assert stats["skipped"] > 0 and stats["pack_count"] == 0      # host tensors have nowhere to be offloaded to
    assert stats["mode"] == "cpu" and stats["min_bytes"] == 64
    mgr = OffloadManager("cpu", min_bytes=64)
    with mgr.training_step():
        (torch.randn(16, 64, requires_grad=True) @ w).sum().backward()
    assert mgr.get_stats()["peak_rss_bytes"] > 0 and mgr.get_stats()["skipped"] > 0
    comp = SavedTensorCompressor("svd", rank=4, min_numel=16)
    low = torch.randn(64, 4) @ torch.randn(4, 32)
    packed = comp.pack(low)
    torch.testing.assert_close(comp.unpack(packed), low, rtol=1e-3, atol=1e-3)
    small = torch.randn(3)
    assert comp.unpack(comp.pack(small)) is small          # below the size floor: passed through


def test_optional_adapters_report_instead_of_raising():
    from stacr_b200.protocols.baselines import actnn_adapter, gact_adapter, torchao_adapter
    from stacr_b200.protocols.baselines._optional import AdapterStatus
    from stacr_b200.protocols.baselines.bnb_optimizer import BNBStatus, estimate_optimizer_savings, try_create_8bit_optimizer

    net = nn.Sequential(nn.Linear(64, 128), nn.Linear(128, 4))
    for adapter, fn in ((actnn_adapter, "try_enable_actnn"), (gact_adapter, "try_enable_gact")):
        model, result = getattr(adapter, fn)(net, "L2")
        assert model is net and result.status in (AdapterStatus.SKIPPED_NOT_INSTALLED, AdapterStatus.SKIPPED_INCOMPATIBLE, AdapterStatus.OK)
        assert isinstance(result.to_dict()["ok"], bool)
    made, result = torchao_adapter.try_create_torchao_optimizer(net.parameters(), "adamw8bit")
    assert (made is None) == (not result.ok)
    res = try_create_8bit_optimizer(net.parameters(), "adamw", prefer="intree")
    assert res.status == BNBStatus.OK_INTREE and res.optimizer is not None
    assert try_create_8bit_optimizer(net.parameters(), "lion", prefer="intree").status == BNBStatus.SKIPPED_UNSUPPORTED_OPTIMIZER
    bnb = try_create_8bit_optimizer(net.parameters(), "adamw", prefer="bnb")
    assert bnb.status in (BNBStatus.SKIPPED_NOT_INSTALLED, BNBStatus.SKIPPED_NO_CUDA, BNBStatus.OK, BNBStatus.ERROR)
    est = estimate_optimizer_savings(net)
    assert 0 < est["int8_state_bytes"] < est["fp32_state_bytes"] and est["savings_ratio"] > 1.0


def test_compression_diagnostics_context_restores_everything():
    import stacr_b200 as S
    from stacr_b200.diagnostics import compression_diagnostics
    from stacr_b200.models import build_model

    torch.manual_seed(0)
    model = build_model("gpt-tiny", n_layer=1).train()
    layers = S.apply_stacr(model, rank=4, min_features=8)
    ids = torch.randint(0, 1024, (2, 16))
    model(input_ids=ids, labels=ids).loss.backward()
    state = {k: v.clone() for k, v in model.state_dict().items()}
    flags = {n: m.training for n, m in model.named_modules()}
    with compression_diagnostics(model):
        assert all(m.p == 0.0 for m in model.modules() if isinstance(m, nn.Dropout))
        S.set_step(layers, 999)
        model(input_ids=ids, labels=ids).loss.backward()
    for k, v in model.state_dict().items():
        assert torch.equal(v, state[k]), k                 # bases, step counters and weights are as before
    assert {n: m.training for n, m in model.named_modules()} == flags


# ------------------------------------------------------------------------------------------------ small protocols
def test_transfer_protocol_pairs_a_dense_and_a_compressed_run():
    from experiments.protocols.openwebtext_transfer import paired_run

    out = paired_run(model_id="gpt-tiny", steps=6, bs=2, seq=32, device="cpu", stacr=dict(rank=4, residual_budget=0.01, turbo_after_step=None, min_features=8))
    assert set(out) >= {"baseline", "stacr", "loss_gap"} and out["wrapped_layers"] > 0
    assert all(v["last_loss"] == v["last_loss"] for v in (out["baseline"], out["stacr"])) and abs(out["loss_gap"]) < 1.0


def test_graph_protocol_trains_and_wraps():
    from experiments.protocols.graph import run

    dense = run(method="baseline", epochs=3, hidden=32)
    wrapped = run(method="stacr", epochs=3, hidden=32, rank=4)
    assert dense["wrapped"] == 0 and wrapped["wrapped"] == 2 and 0.0 <= wrapped["test_accuracy"] <= 1.0


# ------------------------------------------------------------------------------------------------ CLI
def _cli(*args):
    env = {**os.environ, "PYTHONPATH": REPO}
    return subprocess.run([sys.executable, "-m", "stacr", *args], capture_output=True, text=True, env=env, cwd=REPO, timeout=300)


def test_cli_exit_codes_and_override_types(tmp_path):
    ok = _cli("train", "--config", "synthetic_stacr", "--device", "cpu", "--dry-run", "--set", "rank=4", "--set", "residual_mode=none", "--set", "amp=off")
    assert ok.returncode == 0
    cfg = json.loads(ok.stdout)
    assert cfg["rank"] == 4 and cfg["residual_mode"] == "none" and cfg["amp"] == "off"    # 'off' and 'none' stay strings
    assert _cli("train", "--config", "no_such_config").returncode != 0
    assert _cli("train", "--config", "synthetic_stacr", "--set", "rank").returncode != 0
    assert _cli("train", "--config", "synthetic_stacr", "--set", "method=warp").returncode != 0
    fid = _cli("fidelity", "--config", "synthetic_gpt_cpu", "--device", "cpu", "--demo", "--output", str(tmp_path / "fid.csv"))
    assert fid.returncode == 0 and (tmp_path / "fid.csv").is_file() and (tmp_path / "fid.config.json").is_file()
    row = json.loads(fid.stdout)
    assert 0.0 < row["mean_cosine"] <= 1.0 and row["wrapped_layers"] > 0 and row["worst_unwrapped_cosine"] > 0.99
    assert _cli("reproduce", "run", "no-such-profile").returncode != 0
    assert _cli("benchmarks", "run", "pythia", "--dry-run").returncode == 0
    assert _cli("doctor").returncode == 0
