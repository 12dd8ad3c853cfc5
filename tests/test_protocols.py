"""Protocol package on CPU: profile table, runner switches, checkpoint-boundary codec, attention surface, comparators, planners."""

import dataclasses
import json

import pytest
import torch
from torch import nn

from experiments.protocols.__main__ import main as protocol_cli, make_config, profiles
from experiments.protocols.logging import NullLogger, RunLogger
from experiments.protocols.training import (ConvergenceConfig, _adaptive_config, checkpoint_boundary_config, parse_rank_schedule,
                                             run_convergence_experiment)
from stacr_b200.adaptive import STACRConfig, STACRLinear
from stacr_b200.models import build_model
from stacr_b200.protocols.config.training import BaselineConfig

TINY = dict(batch_size=2, max_length=32, max_steps=2, train_examples=8, eval_examples=4, device="cpu", stacr_min_features=8)


def _tiny_model_for(raw):
    name = str(raw.get("model") or ("bert" if raw.get("task") == "sst2" else "gpt2")).lower()
    for key, tiny in (("bert", "bert-tiny"), ("llama", "llama-tiny"), ("qwen", "llama-tiny")):
        if key in name:
            return tiny
    return "gpt-tiny"


# ------------------------------------------------------------------------------------------------ profiles
def test_every_profile_parses_and_groups_are_complete():
    table = profiles()
    assert len(table) >= 122
    groups = {p["group"] for p in table.values()}
    for needed in ("gpt2-medium-quality", "pythia-memory", "pythia-10k", "galore-composition", "bert-sst2", "attention-surface", "mechanism-fidelity",
                   "factorization", "tensor-parallel", "adaptive-runtime", "gradient-accumulation", "matched-bytes-throughput", "layer-fidelity",
                   "theorem-checkpoints", "checkpoint-boundary", "gnn-surface-boundary", "checkpointed-llama", "residual-fidelity", "rank-allocation"):
        assert needed in groups, needed
    for name, prof in table.items():
        cfg = make_config(prof, 42, {})
        assert cfg.run_tag
        if prof["group"] != "smoke":  # the single-rank TP smoke profile shards over one rank on purpose
            assert prof.get("world_size", 1) == (2 if cfg.use_tensor_parallel or cfg.use_ddp else 1), name
    tp = [n for n, p in table.items() if p["group"] == "tensor-parallel"]
    assert len(tp) == 4 and all(table[n]["world_size"] == 2 for n in tp)


# one profile per behaviour that the runner has to support
REPRESENTATIVE = ["gpt2-medium-quality-full", "gpt2-medium-quality-checkpoint", "galore-composition-full", "bert-sst2-full", "attention-surface-joint-qk"
                  if "attention-surface-joint-qk" in profiles() else sorted(n for n, p in profiles().items() if p["group"] == "attention-surface")[-1],
                  "factorization-tt", "factorization-tucker", "factorization-svd", "layer-fidelity-untracked-r8", "residual-controls-bert-sparse-50",
                  "adaptive-gpt2-large-b8-turbo", "gradient-accumulation-full", "matched-bytes-bert-base-lowrank", "rank-allocation-scheduled",
                  "checkpoint-boundary-long-compressed", "surface-boundary-llama-full", "pythia-5k-turbo"]


@pytest.mark.parametrize("name", REPRESENTATIVE)
def test_representative_profiles_train_two_steps_on_tiny_models(name):
    prof = profiles()[name]
    raw = prof["config"]
    over = dict(TINY, model=_tiny_model_for(raw), rank=min(int(raw.get("rank", 8)), 8), grad_fidelity_interval=1, per_layer_grad_fidelity_interval=1,
                activation_spectrum_interval=1, stacr_ckpt_min_numel=0)
    if raw.get("stacr_ckpt_rank"):
        over["stacr_ckpt_rank"] = 8
    if raw.get("stacr_attention_rank"):
        over["stacr_attention_rank"] = 4
    if raw.get("reshape_shape"):
        over["reshape_shape"] = None
    if raw.get("stacr_per_layer_rank_schedule"):
        over["stacr_per_layer_rank_schedule"] = "c_fc=4,c_proj=6"
    final = run_convergence_experiment(make_config(prof, 42, over), NullLogger())
    assert final["status"] == "ok" and final["steps"] == 2
    assert final["train_loss_last"] == final["train_loss_last"]  # finite
    if raw.get("method", "baseline") != "baseline":
        assert final["n_wrapped_layers"] > 0


def test_runner_config_validation_and_engine_mapping():
    names = {f.name for f in dataclasses.fields(ConvergenceConfig)}
    assert len(names) >= 190
    cfg = ConvergenceConfig(method="stacr", stacr_lazy_update=False, stacr_post_warmup_mode="none", stacr_skip_residual=True, stacr_chunk_size=128,
                            stacr_quantize_bits=8, stacr_refresh_period=77)
    eng = _adaptive_config(cfg)
    assert (eng.lazy_update_enabled, eng.post_warmup_residual_mode, eng.skip_residual_enabled, eng.chunk_size, eng.refresh_period) == (False, "none", True, 128, 77)
    assert _adaptive_config(ConvergenceConfig(method="stac")).residual_mode == "none"
    assert ConvergenceConfig(stacr_post_warmup_residual_mode="threshold").stacr_post_warmup_mode == "threshold"
    assert ConvergenceConfig(stacr_use_planner=True, stacr_planner_enforce=True).stacr_planner == "bytes"
    ck = checkpoint_boundary_config(ConvergenceConfig(stacr_ckpt_rank=16, stacr_ckpt_warmup_steps=3, stacr_ckpt_quantize_coefficients=True))
    assert ck.enabled and (ck.rank, ck.warmup_steps, ck.quantize_coefficients) == (16, 3, True)
    assert parse_rank_schedule("c_fc=4, c_proj=12") == {"c_fc": 4, "c_proj": 12} and parse_rank_schedule(None) == {}
    for bad in (dict(method="nope"), dict(use_ddp=True, use_tensor_parallel=True), dict(padding_mode="left"), dict(conv_compression_mode="tucker"),
                dict(stacr_decoder_target_mode="some")):
        with pytest.raises(ValueError):
            ConvergenceConfig(**bad)
    with pytest.raises(ValueError):
        parse_rank_schedule("c_fc")
    with pytest.raises(ValueError):
        ConvergenceConfig.from_raw({"no_such_field": 1})


def test_rank_schedule_and_small_layer_scaling_reach_the_layers():
    cfg = ConvergenceConfig(method="stacr", model="gpt-tiny", rank=8, stacr_per_layer_rank_schedule="c_fc=4,c_proj=6", **TINY)
    from experiments.protocols.training import replace_linear_with_stacr, select_targets

    model = build_model("gpt-tiny")
    layers = replace_linear_with_stacr(model, select_targets(model, cfg), cfg)
    ranks = {l.source_name.rsplit(".", 1)[-1]: l.config.rank for l in layers}
    assert ranks == {"c_fc": 4, "c_proj": 6}
    cfg2 = ConvergenceConfig(method="stacr", model="gpt-tiny", rank=8, stacr_small_layer_rank_scale=0.5, stacr_small_layer_residual_scale=2.0, **TINY)
    model2 = build_model("gpt-tiny")
    layers2 = replace_linear_with_stacr(model2, select_targets(model2, cfg2), cfg2)
    small = [l for l in layers2 if l.in_features < 1024]
    assert small and all(l.config.rank == 4 and l.config.residual_budget == pytest.approx(0.01) for l in small)
    assert all(l.config.rank == 8 for l in layers2 if l.in_features >= 1024)
    mlp_only = ConvergenceConfig(method="stacr", stacr_surface="mlp+attention", stacr_decoder_target_mode="attention_only", **TINY)
    assert all(".attn." in n for n in select_targets(build_model("gpt-tiny"), mlp_only))


def test_baseline_config_forms():
    b = BaselineConfig.from_mapping({"name": "x", "saved_tensors_offload": "cpu", "saved_tensors_offload_min_bytes": 5, "galore": "rank=16,update_gap=7,scale=0.5",
                                     "galore_target_modules": "attn,mlp", "grad_accum_steps": 2})
    assert (b.offload, b.offload_min_bytes, b.saved_tensors_offload) == ("cpu", 5, "cpu")
    assert b.galore_options() == {"rank": 16, "update_proj_gap": 7, "scale": 0.5, "target_modules": ["attn", "mlp"]}
    assert "accum=2" in b.get_description() and not b.is_default()
    assert BaselineConfig().is_default() and BaselineConfig().galore_options() is None
    assert BaselineConfig.from_legacy("checkpointing").checkpointing == "transformer_hf"
    assert BaselineConfig.from_legacy("galore").galore.startswith("rank=128")
    combo = BaselineConfig.from_legacy("bf16+8bit+offload+c1")
    assert (combo.amp, combo.optimizer_8bit, combo.offload, combo.c1_checkpoint_compression) == ("bf16", True, "cpu", True)
    with pytest.raises(ValueError):
        BaselineConfig.from_mapping({"bogus": 1})
    with pytest.raises(ValueError):
        BaselineConfig.from_legacy("warp-drive")
    with pytest.raises(ValueError):
        BaselineConfig(galore="rank").galore_options()


def test_gradient_accumulation_consumes_microbatches_and_matches_big_batch():
    """Two micro-batches of 2 with accumulation give the same first update as one batch of 4 (dense model, no dropout)."""
    base = dict(model="gpt-tiny", method="baseline", max_length=16, max_steps=1, train_examples=4, eval_examples=2, device="cpu", lr=1e-3, warmup_ratio=0.0,
                model_overrides={"resid_pdrop": 0.0, "embd_pdrop": 0.0, "attn_pdrop": 0.0})
    a = run_convergence_experiment(ConvergenceConfig(batch_size=4, **base), NullLogger())
    b = run_convergence_experiment(ConvergenceConfig(batch_size=2, baseline_cfg={"grad_accum_steps": 2}, **base), NullLogger())
    assert a["status"] == b["status"] == "ok"
    assert b["train_loss_last"] == pytest.approx(a["train_loss_last"], rel=1e-4)


# ------------------------------------------------------------------------------------------------ CLI and logger
def test_protocol_cli_list_dry_run_world_size_and_run(tmp_path, capsys):
    assert protocol_cli(["list", "--group", "tensor-parallel"]) == 0
    assert capsys.readouterr().out.count("world=2") == 4
    assert protocol_cli(["run", "pythia-memory-full", "--dry-run", "--seeds", "7", "--set", "rank=4"]) == 0
    plan = json.loads(capsys.readouterr().out)
    assert plan["seeds"] == [7] and plan["configs"][0]["rank"] == 4 and plan["configs"][0]["seed"] == 7
    assert protocol_cli(["run", "tensor-parallel-full", "--steps", "1"]) == 2  # needs two ranks
    args = ["run", "smoke-tiny-full", "--steps", "2", "--seeds", "1", "--device", "cpu", "--output", str(tmp_path)]
    assert protocol_cli(args) == 0
    run_dir = tmp_path / "smoke-tiny-full" / "seed1"
    final = json.loads((run_dir / "final.json").read_text())
    assert final["status"] == "ok" and (run_dir / "config.json").is_file()
    assert len((run_dir / "metrics.jsonl").read_text().strip().splitlines()) == 2
    with pytest.raises(SystemExit):
        protocol_cli(["run", "no-such-profile"])


def test_run_logger_files(tmp_path):
    log = RunLogger(tmp_path / "r")
    log.write_config({"a": 1})
    log.log({"step": 0, "loss": 1.0})
    log.write_final({"status": "ok"})
    assert json.loads((tmp_path / "r" / "config.json").read_text()) == {"a": 1}
    assert json.loads((tmp_path / "r" / "metrics.jsonl").read_text().splitlines()[0])["loss"] == 1.0
    NullLogger().log({"x": 1})


# ------------------------------------------------------------------------------------------------ checkpoint-boundary codec
def test_boundary_codec_roundtrip_fallbacks_and_state():
    from stacr_b200.protocols.checkpointing import CheckpointBoundaryCodec, STACRCheckpointSpec

    torch.manual_seed(0)
    spec = STACRCheckpointSpec(site_id="b0", module_type="Block", model_family="gpt2", hidden_size=32, rank=8, warmup_steps=0, min_numel=0,
                               refresh_trigger="off")
    codec = CheckpointBoundaryCodec(spec)
    low = torch.randn(4, 16, 8) @ torch.randn(8, 32)          # exactly rank 8
    rec = codec.pack_tensor(low, training=True)
    assert not rec.is_dense_fallback and rec.coeff.shape == (64, 8)
    assert torch.allclose(codec.unpack_record(rec), low, atol=1e-3, rtol=1e-3)
    assert codec.pack_count == 1 and codec.unpack_count == 1 and codec.basis_initialized
    assert codec.pack_tensor(low, training=False).is_dense_fallback          # evaluation keeps the tensor
    assert codec.pack_tensor(torch.randn(4, 16, 31), training=True).is_dense_fallback  # not a boundary of this site
    bad = low.clone()
    bad[0, 0, 0] = float("nan")
    assert codec.pack_tensor(bad, training=True).is_dense_fallback and codec.fallbacks.get("input_nonfinite") == 1
    q = CheckpointBoundaryCodec(dataclasses.replace(spec, quantize_coefficients=True))
    recq = q.pack_tensor(low, training=True)
    assert recq.coeff_quantized and recq.coeff.dtype == torch.int8
    err = (q.unpack_record(recq) - low).norm() / low.norm()
    assert err < 0.02
    clone = CheckpointBoundaryCodec(spec)
    clone.load_state_dict(codec.state_dict())
    assert clone.basis_initialized and torch.equal(clone.basis, codec.basis)
    stats = codec.stats()
    assert stats["packs"] >= 1 and 0 < stats["stored_bytes"] < stats["raw_bytes"]


def test_boundary_checkpointing_gradients_match_dense_when_boundary_is_low_rank():
    from stacr_b200.protocols.checkpointing import STACRCheckpointConfig, enable_c1_checkpointing_for_model

    torch.manual_seed(0)
    model = build_model("gpt-tiny", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0).train()
    hidden = model.config.n_embd
    ids = torch.randint(0, model.config.vocab_size, (2, 16))
    model(input_ids=ids, labels=ids).loss.backward()
    ref = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad(set_to_none=True)
    runtime = enable_c1_checkpointing_for_model(model, STACRCheckpointConfig(enabled=True, rank=hidden, warmup_steps=0, min_numel=0))  # full rank: lossless
    model(input_ids=ids, labels=ids).loss.backward()
    for n, p in model.named_parameters():
        if n in ref:
            assert torch.allclose(p.grad, ref[n], atol=2e-4, rtol=2e-3), n
    stats = runtime.stats()
    assert runtime.is_active and len(stats["sites"]) == model.config.n_layer and stats["raw_bytes"] > 0
    with pytest.raises(ValueError):
        enable_c1_checkpointing_for_model(nn.Linear(4, 4), STACRCheckpointConfig(enabled=True))


# ------------------------------------------------------------------------------------------------ attention surface
def test_attention_surface_joint_qk_mask_awareness_and_split():
    from stacr_b200.protocols.attention import (JointQKSTACRLinear, _extract_token_mask, _MaskAwareSTACRLinear, apply_stacr_to_attention,
                                                clear_joint_qk_bases)

    torch.manual_seed(0)
    clear_joint_qk_bases()
    conf = STACRConfig(rank=4, residual_mode="topk", update_trigger="fixed", update_interval=1)
    bert = build_model("bert-tiny").train()
    report = apply_stacr_to_attention(bert, conf, mask_aware=True, joint_qk=True)
    layers = bert.config.num_hidden_layers
    assert report.joint_qk_pairs == layers and report.replaced == 3 * layers
    attn = bert.bert.encoder.layer[0].attention.self
    assert isinstance(attn.query, _MaskAwareSTACRLinear) and isinstance(attn._joint_qk_wrapper, JointQKSTACRLinear)
    ids = torch.randint(0, bert.config.vocab_size, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[1, 8:] = 0
    out = bert(input_ids=ids, attention_mask=mask, labels=torch.tensor([0, 1]))
    out.loss.backward()
    q_inner, k_inner = attn.query.inner, attn.key.inner
    assert q_inner._resolve_basis().data_ptr() == k_inner._resolve_basis().data_ptr()  # one pooled basis for the pair
    assert attn.query.inner.linear.weight.grad is not None
    add = torch.zeros(2, 1, 1, 12)
    add[1, ..., 8:] = -1e4
    keep = _extract_token_mask(add, 12, torch.device("cpu"))
    assert keep.tolist() == mask.bool().tolist()
    assert _extract_token_mask(torch.ones(2, 5), 12, torch.device("cpu")) is None
    gpt = build_model("gpt-tiny").train()
    skipped = apply_stacr_to_attention(gpt, conf)
    assert skipped.replaced == 0 and skipped.skipped == gpt.config.n_layer and skipped.warnings
    split = apply_stacr_to_attention(gpt, conf, enable_gpt2_c_attn_split=True)
    assert split.replaced == 3 * gpt.config.n_layer
    w = gpt.transformer.h[0].attn.c_attn.source.weight
    ids = torch.randint(0, gpt.config.vocab_size, (2, 8))
    gpt(input_ids=ids, labels=ids).loss.backward()
    assert w.grad is not None and w.grad.abs().sum() > 0   # the fused parameter keeps training
    adaptive_rank = apply_stacr_to_attention(build_model("bert-tiny"), STACRConfig(rank=4, rank_mode="variance"), joint_qk=True)
    assert adaptive_rank.joint_qk_pairs == 0 and any("joint_qk" in w for w in adaptive_rank.warnings)
    clear_joint_qk_bases()


# ------------------------------------------------------------------------------------------------ comparators
def test_factor_codecs_and_compressed_linear_gradients():
    from stacr_b200.protocols.compression import Compressor
    from stacr_b200.protocols.layers import CompressedLinear

    torch.manual_seed(0)
    x = torch.randn(16, 4) @ torch.randn(4, 24)
    assert torch.allclose(Compressor.decompress_svd(Compressor.compress_svd_factors(x, 4)), x, atol=1e-4)
    tt = Compressor.compress_tt_factors(x, (4, 4, 4, 6), 16)
    assert torch.allclose(Compressor.decompress_tt(tt).reshape(16, 24), x, atol=1e-3)
    tk = Compressor.compress_tucker_factors(x, (4, 4, 4, 6), [4, 4, 4, 6])
    assert torch.allclose(Compressor.decompress_tucker(tk).reshape(16, 24), x, atol=1e-3)
    q8 = Compressor.dequantize_svd_factors(Compressor.quantize_svd_factors(Compressor.compress_svd_factors(x, 4), bits=8))
    assert (Compressor.decompress_svd(q8) - x).norm() / x.norm() < 0.05
    lin = nn.Linear(24, 8)
    inp = x.clone().requires_grad_(True)
    lin(inp).square().sum().backward()
    gw, gx = lin.weight.grad.clone(), inp.grad.clone()
    lin.zero_grad()
    comp = CompressedLinear.from_linear(lin, {"method": "svd", "rank": 4})
    inp2 = x.clone().requires_grad_(True)
    comp(inp2).square().sum().backward()
    assert torch.allclose(inp2.grad, gx, atol=1e-5)                       # input gradient is exact
    assert torch.allclose(comp.linear.weight.grad, gw, atol=1e-3, rtol=1e-3)     # rank-4 input: the weight gradient is too
    with pytest.raises(ValueError):
        CompressedLinear.from_linear(lin, {"method": "wavelet", "rank": 4})


def test_prac_projection_is_seeded_per_window_and_unbiased_enough():
    from stacr_b200.protocols.prac import PRACConfig, replace_linear_with_prac, set_prac_global_step

    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 4))
    layers = replace_linear_with_prac(net, ["0"], PRACConfig(rank=16, update_proj_gap=5, quiet=True))
    layer = layers[0]
    p0 = layer.projection.clone()
    set_prac_global_step(net, 4)
    assert torch.equal(layer.projection, p0)
    set_prac_global_step(net, 5)
    assert not torch.equal(layer.projection, p0)
    set_prac_global_step(net, 0)
    assert torch.equal(layer.projection, p0)            # the window seed is a pure function of (seed, name, window)
    x = torch.randn(8, 64, requires_grad=True)
    net.train()
    net(x).sum().backward()
    assert layer.linear.weight.grad.shape == (32, 64) and x.grad is not None
    net.eval()
    assert torch.allclose(net(x), nn.Sequential(layer.linear, net[1], net[2])(x))


def test_basis_control_comparators_and_lowrank_optimizers():
    from stacr_b200.comparators.activation import OasisLinear, UntrackedLinear
    from stacr_b200.comparators.galore_adapter import create_galore_optimizer
    from stacr_b200.comparators.subtrack_adapter import create_subtrack_optimizer

    torch.manual_seed(0)
    for cls in (UntrackedLinear, OasisLinear):
        layer = cls.from_linear(nn.Linear(32, 16), rank=4)
        layer.train()
        x = torch.randn(10, 32, requires_grad=True)
        ref = torch.nn.functional.linear(x, layer.weight, layer.bias)
        out = layer(x)
        assert torch.allclose(out, ref, atol=1e-6)
        out.sum().backward()
        assert layer.weight.grad is not None and bool(layer.basis_ready)
        q = layer.basis.float()
        assert torch.allclose(q.t() @ q, torch.eye(4), atol=1e-4)
    factories = (lambda net: create_galore_optimizer(net, lr=1e-2, rank=4, update_proj_gap=2, target_modules=["0"]),
                 lambda net: create_subtrack_optimizer(net, {"lr": 1e-2, "subtrack_rank": 4, "subtrack_update_interval": 4, "subtrack_target_modules": ["0"]}))
    for factory in factories:
        net = nn.Sequential(nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 2))
        opt = factory(net)
        x, y = torch.randn(32, 16), torch.randn(32, 2)
        first = None
        for _ in range(12):
            opt.zero_grad()
            loss = (net(x) - y).square().mean()
            loss.backward()
            opt.step()
            first = first if first is not None else float(loss)
        assert float(loss) < first


# ------------------------------------------------------------------------------------------------ planners and byte accounting
def test_layer_planner_keeps_only_layers_that_save_bytes():
    from stacr_b200.protocols.planner import plan_stacr_layers, summarize_layer_decisions

    model = build_model("gpt-tiny")
    cfg = ConvergenceConfig(method="stacr", model="gpt-tiny", rank=4, **TINY)
    names = [n for n, m in model.named_modules() if n.endswith(("c_fc", "mlp.c_proj"))]
    decisions = plan_stacr_layers(model, cfg, names)
    assert len(decisions) == len(names) and all(d.keep == (d.net_bytes > 0) or d.forced for d in decisions)
    assert all(d.net_bytes == d.saved_activation_bytes - d.stacr_stored_bytes for d in decisions)
    summary = summarize_layer_decisions(decisions)
    assert summary["candidates"] == len(names) and summary["kept"] == sum(d.keep for d in decisions) and sum(summary["reasons"].values()) == len(names)
    fat = ConvergenceConfig(method="stacr", model="gpt-tiny", rank=64, stacr_residual_budget=0.9, stacr_quantize_residuals=False, **TINY)
    assert not any(d.keep for d in plan_stacr_layers(model, fat, names))
    forced = ConvergenceConfig(method="stacr", model="gpt-tiny", rank=64, stacr_residual_budget=0.9, stacr_quantize_residuals=False,
                               stacr_force_compress_layers=names[0], **TINY)
    assert [d.name for d in plan_stacr_layers(model, forced, names) if d.keep] == [names[0]]


def test_memory_accounting_closed_forms():
    import stacr_b200.memory_accounting as M

    assert M.original_bytes((8, 16), torch.float16) == 256
    assert M.svd_stored_elements(100, 50, 5) == 100 * 5 + 5 + 5 * 50
    r = M.svd_rank_from_budget(100, 50, torch.float32, budget_bytes=4000, include_meta=False)
    assert M.svd_stored_bytes(100, 50, r, torch.float32, include_meta=False).total_bytes <= 4000 < M.svd_stored_bytes(100, 50, r + 1, torch.float32, include_meta=False).total_bytes
    assert M.tt_uniform_ranks([4, 5, 6], 3) == [1, 3, 3, 1] and M.tt_stored_elements([4, 5, 6], [1, 3, 3, 1]) == 4 * 3 + 3 * 5 * 3 + 3 * 6
    assert M.validate_tt_ranks([4, 5, 6], [1, 3, 3, 1])[0] and not M.validate_tt_ranks([4, 5, 6], [2, 3, 3, 1])[0]
    assert M.tucker_stored_elements([4, 5, 6], [2, 2, 2]) == 8 + 8 + 10 + 12
    assert M.validate_tucker_ranks([4, 5], [4, 5])[0] and not M.validate_tucker_ranks([4, 5], [5, 5])[0]
    plan = M.plan_svd(512, 256, torch.float16, target_ratio=8.0)
    assert plan.feasible and plan.achieved_ratio >= 8.0
    assert not M.plan_svd(4, 4, torch.float16, target_ratio=1000.0).feasible
    full = M.stacr_stored_bytes(1024, 512, 8, residual_budget=0.005, dtype=torch.float16, coeff_bits=8, residual_bits=4)
    lowrank = M.stacr_stored_bytes(1024, 512, 8, residual_budget=0.0, dtype=torch.float16, coeff_bits=8)
    assert lowrank.total_bytes < full.total_bytes < M.original_bytes((1024, 512), torch.float16)
    assert M.stacr_rho_max(1024, 512, torch.float16) > 1.0


def test_reconstruction_oracles_and_drift_tracker():
    import torch

    import stacr_b200 as S
    from experiments.protocols.diagnostics import (C1DriftTracker, reconstruct_stacr_activation, reconstruct_svd_lowrank, reconstruction_metrics,
                                                   reconstruction_report)

    torch.manual_seed(0)
    base = torch.randn(256, 4) @ torch.randn(4, 64)
    x = base + 0.05 * torch.randn(256, 64)
    lin = torch.nn.Linear(64, 32)
    layer = S.STACRLinear.from_linear(lin, rank=4, residual_budget=0.02, residual_bits=8)
    layer.train()
    same, info = reconstruct_stacr_activation(layer, x)
    assert info["reconstruction_scope"] == "baseline_or_uninitialized_basis" and same is x
    layer.set_step(0)
    layer(x).sum().backward()
    rec, info = reconstruct_stacr_activation(layer, x)
    m = reconstruction_metrics(x, rec)
    assert info["rank"] == 4 and info["residual_entries_kept"] == int(round(0.02 * x.numel())) and info["residuals_quantized"]
    assert m["relative_error"] < 0.2 and m["cosine"] > 0.98
    srec, sinfo = reconstruct_svd_lowrank(x, 4)
    assert sinfo["rank"] == 4 and reconstruction_metrics(x, srec)["relative_error"] < 0.2
    model = torch.nn.Sequential(layer)
    report = reconstruction_report(model, [layer], lambda: model(x))
    assert report["summary"]["count"] == 1 and report["layers"][0]["layer"] == "0"
    # drift: flat energies and losses, then one site's energy jumps while the loss worsens
    tracker = C1DriftTracker(window=4)
    stats = lambda e: {"sites": {"blk0": {"packs": 3, "last_residual_energy": 0.05}, "blk1": {"packs": 3, "last_residual_energy": e}}}
    for step in range(6):
        out = tracker.update(stats(0.06), global_step=step, optimizer_step=step, loss_value=2.0)
        assert out["signal"] is None and out["sites_tracked"] == 2
    out = tracker.update(stats(0.30), global_step=6, optimizer_step=6, loss_value=2.5)
    assert out["signal"] == "fast" and out["leading_site"] == "blk1"
    event = tracker.summary()["first_finite_drift_event"]
    assert event["site"] == "blk1" and event["global_step"] == 6 and event["energy_ratio"] > 4
    assert tracker.update(stats(0.30), global_step=7, optimizer_step=7, loss_value=float("nan"))["finite"] is False


def test_data_parallel_arm_reports_why_it_cannot_run_on_this_host():
    from experiments.protocols.training import ConvergenceConfig, data_parallel_blockers

    cfg = ConvergenceConfig(task="sst2", use_data_parallel=True)
    why = data_parallel_blockers(cfg, "cpu")
    assert "non-CUDA device" in why and "fewer than 2 CUDA devices" in why
