"""Comparator packages (PRAC compressor, INSTANT, SubTrack protocol), protocol helpers, per-grid entry modules, top-level scripts."""

import importlib
import json
import os
import subprocess
import sys
from types import SimpleNamespace as NS

import pytest
import torch
from torch import nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY_GPT = {"n_layer": 2, "n_embd": 64, "n_head": 2, "vocab_size": 128}
TINY_BERT = {"num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 2, "intermediate_size": 128, "vocab_size": 128}


def test_comparators_alias_resolves_to_the_same_modules():
    import comparators.prac as a
    import stacr_b200.comparators.prac as b
    from comparators.galore_adapter import galore_available  # noqa: F401
    from comparators.per_batch_factors import factorization_benchmark  # noqa: F401

    assert a is b


def test_prac_compressor_is_deterministic_and_an_unbiased_scale():
    from stacr_b200.comparators.prac import PRACCompressor, PRACConfig

    x = torch.randn(32, 256)
    c1, c2 = PRACCompressor(PRACConfig(rank=16, seed=3)), PRACCompressor(PRACConfig(rank=16, seed=3))
    assert torch.equal(c1.reconstruct(x), c2.reconstruct(x))
    assert not torch.equal(c1.reconstruct(x), PRACCompressor(PRACConfig(rank=16, seed=4)).reconstruct(x))
    p = c1.projection(256, x.device, x.dtype)
    assert p.shape == (256, 16)
    assert abs(float(p.square().sum()) / 256 - 1.0) < 0.2          # E[P P^T] = I  =>  ||P||_F^2 ~ features
    assert c1.reconstruct(x.reshape(4, 8, 256)).shape == (4, 8, 256)
    assert c1.stored_bytes(x) == 32 * 16 * 4
    assert c1.projection(300, x.device, x.dtype).shape == (300, 16) and PRACCompressor(PRACConfig(rank=999)).projection(8, "cpu", torch.float32).shape == (8, 8)


def test_instant_energy_basis_counts_and_scale():
    from stacr_b200.comparators.instant.svd import SVD_expected_value, energy_basis

    u = torch.linalg.qr(torch.randn(32, 32)).Q
    spectrum = torch.tensor([10.0, 5.0, 1.0] + [1e-3] * 29)
    gram = u @ torch.diag(spectrum) @ u.t()
    basis = energy_basis(gram, var=0.9, oversample=0)
    assert basis.shape[0] == 32 and 1 <= basis.shape[1] <= 4
    full = energy_basis(gram, var=1.0, oversample=100)
    assert full.shape == (32, 32)
    assert torch.allclose(full @ full.t(), torch.eye(32), atol=1e-4)      # nothing dropped: exact projector
    assert torch.equal(SVD_expected_value(gram, 0.9, 0), basis)


def test_instant_linear_matches_dense_when_subspace_is_complete_and_compresses_otherwise():
    from stacr_b200.comparators.instant import InstantLinear, register_filter, update_compression

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 24), nn.GELU(), nn.Linear(24, 8))
    ref = [p.detach().clone() for p in model.parameters()]
    x = torch.randn(3, 10, 16, requires_grad=True)
    model(x).square().sum().backward()
    want = [p.grad.clone() for p in model.parameters()] + [x.grad.clone()]
    model.zero_grad()
    x.grad = None
    register_filter(model, ["0", "2"])
    assert isinstance(model[0], InstantLinear) and all(torch.equal(a, b) for a, b in zip(ref, model.parameters()))
    eye = torch.eye(10)
    update_compression(model, {"0": eye, "2": eye}, {"0": eye, "2": eye})
    model.train()
    model(x).square().sum().backward()
    got = [p.grad for p in model.parameters()] + [x.grad]
    for a, b in zip(want, got):
        assert torch.allclose(a, b, atol=1e-4)
    # a 4-dimensional token subspace keeps 4 rows per sample
    p4 = torch.linalg.qr(torch.randn(10, 4)).Q
    update_compression(model, {"0": p4, "2": p4}, {"0": p4, "2": p4})
    assert model[0].saved_rows(10) == 4 and model[0].saved_rows(11) == 11
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(tuple(t.shape)) or t, lambda t: t):
        model[0](torch.randn(3, 10, 16, requires_grad=True))
    assert (3, 4, 16) in saved and (3, 10, 16) not in saved
    model.eval()
    assert torch.allclose(model[0](x), nn.functional.linear(x, model[0].weight, model[0].bias))


def test_instant_calibrator_and_training_scripts(tmp_path):
    from stacr_b200.comparators.instant import train_classification, train_language
    from stacr_b200.comparators.instant.model import freeze_layers, get_svd_layers
    from stacr_b200.models import build_model

    model = build_model("gpt2", **TINY_GPT)
    names = get_svd_layers(model, "gpt2")
    assert names and all("lm_head" not in n and "wte" not in n for n in names)
    freeze_layers(model, 1, "gpt2")
    assert all(p.requires_grad == (".h.1." in n or "ln_f" in n or "lm_head" in n) for n, p in model.named_parameters() if ".h." in n or "ln_f" in n)
    out = train_language.main(["--compress", "--synthetic", "--max-steps", "4", "--calib_iter", "2", "--calib_batches", "1", "--max-length", "32",
                               "--batch-size", "2", "--output_dir", str(tmp_path / "lm"), "--device", "cpu", "--model-overrides", json.dumps(TINY_GPT)])
    assert out["method"] == "instant" and out["compressed_layers"] == 8 and 0 < out["mean_saved_row_fraction"] <= 1
    assert (tmp_path / "lm" / "result.json").exists() and (tmp_path / "lm" / "svd_shapes.json").exists()
    dense = train_language.main(["--synthetic", "--max-steps", "2", "--max-length", "32", "--batch-size", "2", "--output_dir", str(tmp_path / "d"),
                                 "--device", "cpu", "--model-overrides", json.dumps(TINY_GPT)])
    assert dense["method"] == "dense" and dense["mean_saved_row_fraction"] == 1.0
    cls = train_classification.main(["--compress", "--max-steps", "3", "--calib_iter", "2", "--calib_batches", "1", "--max-length", "16", "--batch-size", "4",
                                     "--output_dir", str(tmp_path / "c"), "--device", "cpu", "--model-overrides", json.dumps(TINY_BERT)])
    assert 0.0 <= cls["val_accuracy"] <= 1.0 and cls["compressed_layers"] > 0


def test_instant_wrapper_runs_a_command():
    from stacr_b200.comparators.instant_wrapper import run_instant

    assert run_instant([sys.executable, "-c", "raise SystemExit(3)"]) == 3
    with pytest.raises(ValueError):
        run_instant([])


def test_subtrack_adapter_source_selection(tmp_path, monkeypatch):
    from stacr_b200.comparators import subtrack_adapter as A

    monkeypatch.delenv(A.SUBTRACK_SOURCE_ENV, raising=False)
    assert A.activate_subtrack_source() is None and A.subtrack_available() and A.subtrack_revision() == "in-tree"
    A.require_subtrack()
    A.require_pinned_subtrack()
    monkeypatch.setenv(A.SUBTRACK_SOURCE_ENV, str(tmp_path))
    with pytest.raises(RuntimeError, match="complete SubTrack checkout"):
        A.activate_subtrack_source()
    (tmp_path / "low_rank_torch").mkdir()
    (tmp_path / "low_rank_torch" / "__init__.py").write_text("")
    (tmp_path / "utils").mkdir()
    (tmp_path / "utils" / "file_utils.py").write_text("")
    monkeypatch.setattr(sys, "path", list(sys.path))
    assert A.activate_subtrack_source() == tmp_path.resolve() and str(tmp_path.resolve()) in sys.path
    with pytest.raises(RuntimeError, match="needs revision"):       # not a git checkout at the pinned commit
        A.require_pinned_subtrack()
    sys.modules.pop("low_rank_torch", None)


def test_subtrack_protocol_four_arms(tmp_path):
    from stacr_b200.comparators import subtrack_protocol as P

    base = ["--max_train_steps", "4", "--max_length", "16", "--per_device_train_batch_size", "4", "--train_examples", "16", "--eval_examples", "8",
            "--device", "cpu", "--output_dir", str(tmp_path), "--model_overrides", json.dumps(TINY_BERT)]
    plain = P.main(base)
    assert plain["optimizer"] == "adamw" and not plain["stacr"]
    sub = P.main(base + ["--enable_low_rank", "--lora_r", "4"])
    both = P.main(base + ["--enable_low_rank", "--low_rank_method", "galore", "--lora_r", "4", "--enable_stacr", "--stacr_rank", "4"])
    assert sub["optimizer"] == "subtrack" and both["optimizer"] == "galore" and both["stacr_layers"] == 2
    assert sub["optimizer_state_bytes"] < plain["optimizer_state_bytes"]
    assert json.loads((tmp_path / "all_results.json").read_text())["stacr"] is True
    with pytest.raises(ValueError):
        P.main(base + ["--enable_stacr", "--model_name_or_path", "gpt2"])


def test_protocol_helpers_targets_shapes_and_estimators():
    from experiments.protocols import training as T

    assert T.auto_reshape_shape(768) == (8, 8, 12) and T.auto_reshape_shape(1536) == (16, 12, 8) and T.auto_reshape_shape(7) is None
    model = T.create_gpt2_lm("gpt2", **TINY_GPT)
    every = T.get_compression_targets_gpt2(model)
    wide = T.get_compression_targets_gpt2(model, "largest_mlp_only")
    assert len(every) == 4 and wide == [n for n in every if n.endswith("c_proj")]
    with pytest.raises(ValueError):
        T.get_compression_targets_gpt2(model, "bogus")
    bert = T.create_bert_sst2(**TINY_BERT)
    assert T.get_compression_targets_bert(bert) == ["bert.encoder.layer.0.output.dense", "bert.encoder.layer.1.output.dense"]
    cfg = T.ConvergenceConfig(task="wikitext103", model="gpt2", batch_size=2, max_length=16, method="stacr", rank=4, train_examples=8, eval_examples=4)
    train, val, _ = T.setup_wikitext_data(cfg, 128)
    assert len(train) == 4 and train[0]["input_ids"].shape == (2, 16) and len(val) == 2
    sst = T.setup_sst2_data(T.ConvergenceConfig(task="sst2", batch_size=4, max_length=8, train_examples=8, eval_examples=4), 128)
    assert sst[0][0]["labels"].shape == (4,)
    assert T.estimate_storage_for_stacr(model, cfg) is None
    T.replace_linear_with_stacr(model, T.select_targets(model, cfg), cfg)
    est = T.estimate_storage_for_stacr(model, cfg)
    assert est["layers"] > 0 and est["achieved_ratio"] > 1 and est["batch_tokens_est"] == 32
    assert T.estimate_storage_for_stacr(model, cfg, actual_batch_tokens=100)["batch_tokens_est"] == 100
    opt = torch.optim.AdamW(model.parameters(), 1e-3)
    cfg.max_steps = 3
    out = T.train_epoch(model, train, None, opt, None, torch.device("cpu"), cfg, 0, None)
    assert out["steps_completed"] == 3 and out["total_tokens"] == 3 * 32
    out = T.train_epoch(model, train, None, opt, None, torch.device("cpu"), cfg, 1, None, global_step_offset=3)
    assert out["steps_completed"] == 0
    assert T.measure_memory_for_cap() is None or T.measure_memory_for_cap() >= 0
    assert "peak_allocated_bytes" in T.log_memory_complete(None, 0)
    state = T.BaselineState.from_mapping({"amp": 1, "offload": None})
    assert state.amp_manager == 1 and state.status == "enabled"


def test_min_adaptation_rule_switches_init_only_when_the_basis_cannot_adapt():
    from experiments.protocols.training import apply_min_adaptation_rule

    def cfg(**kw):
        return NS(**{"use_random_qr_init": True, "freeze_basis_after_warmup": True, "warmup_steps": 2, "min_adaptation_steps": 10,
                     "allow_unadapted_random_qr": False, **kw})

    with pytest.warns(UserWarning):
        assert apply_min_adaptation_rule(cfg(), 100, log_fn=None).use_random_qr_init is False
    assert apply_min_adaptation_rule(cfg(warmup_steps=50), 100).use_random_qr_init is True
    assert apply_min_adaptation_rule(cfg(freeze_basis_after_warmup=False), 100).use_random_qr_init is True
    assert apply_min_adaptation_rule(cfg(allow_unadapted_random_qr=True), 100).use_random_qr_init is True
    assert apply_min_adaptation_rule(cfg(), None).use_random_qr_init is True


def test_storage_estimators_for_factor_prac_and_boundary_sites():
    from experiments.protocols import training as T
    from stacr_b200.protocols.checkpointing import build_stacr_checkpoint_config, clear_active_c1_runtime, register_c1_sites

    cfg = T.ConvergenceConfig(task="wikitext103", model="gpt2", batch_size=2, max_length=16, method="svd", rank=4)
    model = T.create_gpt2_lm("gpt2", **TINY_GPT)
    T.replace_linear_with_compressed(model, T.get_compression_targets_gpt2(model), cfg)
    est = T.estimate_storage_for_model(model, cfg)
    assert est["layers"] == 4 and est["stored_bytes"] < est["original_bytes"]
    cfg.method = "baseline"
    assert T.estimate_storage_for_model(model, cfg) is None
    from stacr_b200.protocols.prac import PRACConfig, replace_linear_with_prac

    model = T.create_gpt2_lm("gpt2", **TINY_GPT)
    replace_linear_with_prac(model, T.get_compression_targets_gpt2(model), PRACConfig(rank=4, quiet=True))
    est = T.estimate_storage_for_prac(model, cfg)
    assert est["layers"] == 4 and est["persistent_projection_bytes"] > 0 and abs(est["achieved_ratio"] - (2 * 64 / 4 + 2 * 256 / 4) / 4) < 1e-6
    run = NS(stacr_compress_checkpoint=True, stacr_ckpt_rank=8, stacr_ckpt_planner="heuristic", stacr_ckpt_quantize_coefficients=True,
             batch_size=2, max_length=16, baseline_cfg=NS(amp="none"))
    ck = build_stacr_checkpoint_config(run)
    assert ck.enabled and ck.rank == 8 and ck.quantize_coefficients and ck.warmup_steps == 500
    model = T.create_gpt2_lm("gpt2", **TINY_GPT)
    runtime = register_c1_sites(model, run)
    try:
        assert len(runtime.registry) == 2 and runtime.site_count_total == 2 and runtime.planner_summary["sites"] == 2
        assert runtime.resolve_site(model.transformer.h[0].forward) is not None
        est = T.estimate_storage_for_c1(model, cfg)
        assert est["layers"] == 2 and est["achieved_ratio"] > 1
        run.stacr_ckpt_planner = "enforce"                          # tiny boundaries cannot pay for their basis
        with pytest.raises(ValueError, match="rejected every"):
            register_c1_sites(model, run)
    finally:
        clear_active_c1_runtime(clear_registry=True)


def test_graph_protocol_functions():
    from experiments.protocols.graph import (create_gcn_model, evaluate_gnn, get_compression_targets_gnn, run_graph_experiment,
                                             setup_ogbn_arxiv_data, train_gnn_epoch)
    from experiments.protocols.logging import NullLogger
    from experiments.protocols.training import ConvergenceConfig

    cfg = ConvergenceConfig(task="ogbn-arxiv", method="stacr", epochs=4, max_steps=4, lr=1e-2, rank=8, device="cpu")
    cfg.graph_nodes = 400
    data, split, info = setup_ogbn_arxiv_data(cfg)
    assert info["num_features"] == 128 and info["num_classes"] <= 40 and info["train_size"] + info["val_size"] + info["test_size"] == info["num_nodes"]
    model = create_gcn_model(128, 32, info["num_classes"], 3, 0.5)
    assert get_compression_targets_gnn(model) == ["convs.0.lin", "convs.1.lin", "convs.2.lin"]
    opt = torch.optim.Adam(model.parameters(), 1e-2)
    first = train_gnn_epoch(model, data, split["train"], opt)["loss"]
    for _ in range(10):
        last = train_gnn_epoch(model, data, split["train"], opt)["loss"]
    assert last < first and set(evaluate_gnn(model, data, split)) == {"train_acc", "valid_acc", "test_acc"}
    out = run_graph_experiment(cfg, NullLogger())["results"]
    assert out["wrapped_layers"] == 3 and out["epochs_completed"] == 4 and out["activation_ratio"] > 1
    cfg.method = "svd"
    with pytest.raises(ValueError):
        run_graph_experiment(cfg, NullLogger())


def test_optional_adapter_records_and_galore_status_surface(tmp_path):
    from stacr_b200.protocols.baselines import actnn_adapter, gact_adapter, galore_adapter, torchao_adapter

    model = nn.Sequential(nn.Linear(32, 32), nn.Linear(32, 8))
    opt, res = galore_adapter.try_enable_galore(model, rank=4)
    assert opt is not None and res.ok and res.meta["rank"] == 4 and res.details["low_rank_params"] == 2
    assert galore_adapter.check_galore_available()[0] and galore_adapter.check_pytorch_version() == (True, None)
    parsed = galore_adapter.parse_galore_config_string("rank=16, update_gap=50, scale=0.5, type=left")
    assert (parsed.rank, parsed.update_proj_gap, parsed.scale, parsed.proj_type) == (16, 50, 0.5, "left")
    assert galore_adapter.parse_galore_config_string("") is None and galore_adapter.parse_galore_config_string("rank=abc") is None
    assert galore_adapter.create_galore_final_json(res, "o")["status"] == "ok"
    _, skipped = gact_adapter.try_enable_gact(model)
    record = gact_adapter.create_gact_final_json(skipped, str(tmp_path))
    assert record["baseline"] == "gact" and record["status"].startswith("skipped") and record["reason"]
    mock = gact_adapter.MockGACTController(model)
    with mock as m:
        m.iterate()
        m.iterate()
    assert mock.iteration == 2 and not mock.enabled and mock.get_config()["reason"] == "mock_controller"
    ctrl = actnn_adapter.ActNNController(model)
    assert not ctrl.enabled and actnn_adapter.create_actnn_final_json(ctrl.result, "o")["baseline"] == "actnn"
    _, tres = torchao_adapter.try_enable_torchao(model, "bogus")
    assert tres.status.value == "error"
    _, tres = torchao_adapter.try_enable_torchao(model)
    assert not tres.ok and torchao_adapter.create_torchao_final_json(tres, "o")["meta"]["requested_mode"] == "auto"


def test_benchmark_helpers_and_grid_entry_modules():
    from experiments.benchmarks import common, distributed_data, distributed_sharding
    from experiments.benchmarks.registry import EXPERIMENTS
    from stacr_b200.models import build_model

    meta = common.runtime_metadata()
    assert "torch" in meta["versions"] and meta["device"]
    model = build_model("gpt2", **TINY_GPT)
    assert len(common.blocks_of(model)) == 2
    with pytest.raises(RuntimeError):
        common.blocks_of(nn.Linear(2, 2))
    sub = common.restrict_cfg_to_blocks(model, {"surface": "mlp", "min_features": 32, "rank": 4}, lambda i: i == 1)
    assert sub["surface"] == "none" and sub["extra_names"] and all(".h.1." in n for n in sub["extra_names"]) and sub["rank"] == 4
    assert common.freeze_surface_params(model, "mlp", 32) == 8 and not model.transformer.h[0].mlp.c_fc.weight.requires_grad
    rows, handles = common.instrument_rows([model.transformer.h[0].mlp.c_fc])
    ids = torch.randint(0, 128, (2, 8))
    model(input_ids=ids, labels=ids)
    assert list(rows.values()) == [16]
    for h in handles:
        h.remove()
    ppl = common.validation_ppl(model, [{"input_ids": ids, "labels": ids}], amp=False)
    assert 1 < ppl < 1e4 and model.training
    assert distributed_sharding.complement(4)(3) and not distributed_data.complement(4)(8)
    arms = [{"method": "baseline"}, {"method": "turbo_fast"}, ("ckpt_k4", {})]
    os.environ["STACR_SKIP_ARMS"] = "turbo_fast, ckpt_k4"
    try:
        assert distributed_sharding.arm_filter(arms) == [{"method": "baseline"}]
        os.environ["STACR_ARM"] = "nothing"
        with pytest.raises(SystemExit):
            distributed_sharding.arm_filter(arms)
    finally:
        os.environ.pop("STACR_SKIP_ARMS", None)
        os.environ.pop("STACR_ARM", None)
    opt, label, dtype = distributed_sharding.build_opt_honest(model)
    assert label == "torch_adamw_float32_states" and dtype == "torch.float32"
    for name in EXPERIMENTS:
        mod = importlib.import_module(f"experiments.benchmarks.{name}")
        assert callable(mod.main)
        if hasattr(mod, "NAME"):
            assert mod.NAME == name and len(mod.cells()) == len(EXPERIMENTS[name]["cells"])


def test_top_level_experiment_scripts_run_by_path(tmp_path):
    env = dict(os.environ, PYTHONPATH="")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "experiments", "mechanism_replay.py"), "--rows", "32", "--features", "128"],
                         capture_output=True, text=True, cwd=str(tmp_path), env=env, timeout=300)
    assert out.returncode == 0 and "stacr_cosine" in out.stdout and "prac_relative_mse" in out.stdout
    from experiments import composition, evaluate, factorization_benchmark, train

    assert composition.main([])["subtrack_available"] is True
    assert {r["method"] for r in factorization_benchmark.main(["--rows", "16", "--features", "64", "--rank", "2"])} >= {"svd", "tucker", "tt"}
    row = train.main(["--config", "synthetic_stacr", "--steps", "2", "--device", "cpu", "--output", str(tmp_path / "r.csv")])
    assert row["steps"] == 2 and evaluate.main(["--csv", str(tmp_path / "r.csv"), "--columns", "steps", "train_loss"]) == 0
    assert subprocess.run([sys.executable, "-m", "experiments.benchmarks.residual_budget", "--dry-run"], capture_output=True, cwd=ROOT, timeout=300).returncode == 0


def test_nf4_codes_round_trip_and_lora_composition_surface():
    import stacr_b200 as S
    from stacr_b200.models import build_model
    from stacr_b200.protocols.lora import NF4_LEVELS, LoRALinear, NF4Linear, apply_lora, nf4_dequantize, nf4_quantize, trainable_parameter_report

    assert len(NF4_LEVELS) == 16 and NF4_LEVELS[0] == -1.0 and NF4_LEVELS[7] == 0.0 and NF4_LEVELS[-1] == 1.0 and list(NF4_LEVELS) == sorted(NF4_LEVELS)
    torch.manual_seed(0)
    w = torch.randn(40, 96) * 0.05
    back = nf4_dequantize(*nf4_quantize(w), w.shape)
    assert float((back - w).norm() / w.norm()) < 0.12                                  # 16 levels on Gaussian weights
    exact = torch.tensor(NF4_LEVELS).repeat(8)[:64].reshape(1, 64) * 0.5                 # values on the grid survive exactly (up to the 8-bit scale)
    assert torch.allclose(nf4_dequantize(*nf4_quantize(exact), exact.shape), exact, atol=5e-3)
    lin = nn.Linear(96, 40)
    q = NF4Linear(lin)
    assert 4.0 < 8 * q.weight_bytes() / lin.weight.numel() < 4.3 and not any(p.requires_grad for p in q.parameters())
    x = torch.randn(5, 96, requires_grad=True)
    q(x).sum().backward()
    assert torch.allclose(x.grad, q.dequantize().sum(0).expand(5, -1), atol=1e-5)
    adapter = LoRALinear(nn.Linear(16, 8), r=4, alpha=8)
    probe = torch.randn(3, 16)
    assert torch.equal(adapter(probe), adapter.base(probe))                             # B starts at zero: the adapter is a no-op
    adapter.lora_B.data.normal_()
    assert torch.allclose(adapter(probe), nn.functional.linear(probe, adapter.merged_weight(), adapter.base.bias), atol=1e-5)

    model = build_model("gpt2", **TINY_GPT)
    adapters = apply_lora(model)
    report = trainable_parameter_report(model)
    assert len(adapters) == 2 and 0 < report["trainable_pct"] < 10 and report["nf4_weight_bytes"] == 0
    assert all(("lora_" in n) == p.requires_grad for n, p in model.named_parameters())
    assert S.select_target_names(model, surface="mlp", min_features=32) == []           # frozen MLP: empty compression surface
    assert len(S.select_target_names(model, surface="mlp", min_features=32, trainable_only=False)) == 4
    ids = torch.randint(0, 128, (2, 8))
    model(input_ids=ids, labels=ids).loss.backward()
    assert adapters[0].lora_B.grad.abs().sum() > 0 and model.transformer.h[0].mlp.c_fc.weight.grad is None
    bert = build_model("bert-base-uncased", **TINY_BERT)
    assert len(apply_lora(bert, quantize_base=True)) == 4 and trainable_parameter_report(bert)["nf4_weight_bytes"] > 0
    assert isinstance(bert.bert.encoder.layer[0].intermediate.dense, NF4Linear)
    with pytest.raises(ValueError):
        apply_lora(build_model("gpt2", **TINY_GPT), target_modules=["nope"])


def test_fat_storage_control_matches_the_layer_and_saves_more():
    from stacr_b200.comparators.activation import apply_comparator, apply_fat

    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(64, 128), nn.GELU(), nn.Linear(128, 64)).train()

    cfg = dict(rank=4, residual_budget=0.05, surface="all", min_features=1, turbo_after_step=None, residual_bits=8)
    x = torch.randn(3, 16, 64)
    real, lean, fat = make(), make(), make()
    apply_comparator(real, "stacr", cfg)
    apply_fat(lean, cfg, basis_per_call=True, fat_residual=False)
    apply_fat(fat, cfg, basis_per_call=True, fat_residual=True)
    grads = []
    for m in (real, lean, fat):
        m(x).square().sum().backward()
        grads.append([p.grad.clone() for p in m.parameters()])
    for a, b in zip(grads[0], grads[1]):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)               # same factors, same arithmetic
    for a, b in zip(grads[0], grads[2]):
        assert torch.allclose(a, b, rtol=0.05, atol=0.05 * float(a.abs().max()))   # unquantised residual values differ slightly

    def held(model):
        seen = []
        with torch.autograd.graph.saved_tensors_hooks(lambda t: seen.append(t) or t, lambda t: t):
            model[0](x)
        return seen

    fat_saved, lean_saved = held(fat), held(lean)
    assert any(t.dtype == torch.int64 for t in fat_saved) and not any(t.dtype == torch.int64 for t in lean_saved)
    assert all(t.data_ptr() != fat[0].basis.data_ptr() for t in fat_saved)      # a private basis copy per call
    assert sum(t.numel() * t.element_size() for t in fat_saved) > sum(t.numel() * t.element_size() for t in lean_saved)


def test_benchmark_runner_adapter_trace_probe_and_search_helpers():
    from experiments.benchmarks import allocator_stability, capacity_search, common, lora, probes, qlora, rate_distortion, swiglu_surfaces
    from stacr_b200.models import build_model

    over = dict(device="cpu", model_overrides=TINY_GPT)
    old = dict(lora.CFG)
    lora.CFG["min_features"] = 32
    try:
        rows = {(a, s): lora.run_lora("gpt2", 2, 16, 4, 42, a, s, **over) for a in (False, True) for s in (False, True)}
    finally:
        lora.CFG.clear()
        lora.CFG.update(old)
    assert rows[(False, True)]["n_wrapped_layers"] == 4 and rows[(True, True)]["n_wrapped_layers"] == 0
    assert rows[(True, True)]["empty_compression_control"] is True and rows[(True, False)]["n_adapters"] == 2
    with pytest.raises(ValueError):
        lora.run_lora("gpt2", 2, 16, 4, 42, True, False, qlora=True)
    row = qlora.run_qlora("qlora", False, 2, 16, 3, 42, device="cpu", model_overrides=TINY_BERT)
    assert row["quant"] and row["nf4_weight_bytes"] > 0 and row["label_protocol"] == "random_classes" and row["quality_metric_valid"] is False
    assert type(qlora.build("full", device="cpu", **TINY_BERT)).__name__.endswith("ForSequenceClassification")
    stored, dense, n = rate_distortion.payload_bytes("stacr", 4, 0.01, "gpt2", 2, 16, min_features=32, **TINY_GPT)
    assert n == 4 and 0 < stored < dense
    low, _, _ = rate_distortion.payload_bytes("lowrank", 4, 0.01, "gpt2", 2, 16, min_features=32, **TINY_GPT)
    assert low < stored
    best = capacity_search.largest_fitting("gpt2", 16, torch.float32, 1, 3, "baseline", None, steps=2, **over)
    assert best["bs"] == 3
    traced = allocator_stability.trace("stacr_r8", dict(rank=4, surface="mlp", min_features=32, residual_budget=0.01), "gpt2", 2, 16, 12, **over)
    assert [m["step"] for m in traced["marks"]] == [10, 11] and "final_reserved_GiB" in traced
    assert probes.maxlen("gpt2", "baseline", {}, [8, 16], steps=2, measure_from=0, eval_batches=0, **over)["seq"] == 16
    assert probes.one("no-such-model", "t", "baseline", {}, 1, 8, device="cpu", steps=1, measure_from=0) is None      # failure is recorded, not raised
    assert swiglu_surfaces.down_proj_names(build_model("llama-tiny"))[0].endswith("mlp.down_proj")
    cfg = swiglu_surfaces.cfg_for("llama-tiny", "down", {"_down_only": True, "min_features": 32}, 16)
    assert cfg["rank"] == 16 and cfg["surface"] == "none" and cfg["extra_names"] and "_down_only" not in cfg
    sub = common.run_config("sub", model_id="bert-base-uncased", bs=2, seq=8, steps=3, measure_from=0, eval_batches=0, optimizer="subtrack",
                            device="cpu", model_overrides=TINY_BERT)
    assert sub["status"] == "ok" and sub["label_protocol"] == "random_classes"
    g, loss = probes.grads(build_model("gpt2", **TINY_GPT), {"input_ids": torch.randint(0, 128, (1, 8)), "labels": torch.randint(0, 128, (1, 8))}, 7)
    assert loss > 0 and all(v.dtype == torch.float32 for v in g.values())
