"""Trainer, composition, CLI and data-parallel plumbing on CPU (gloo for the two-rank cases)."""

import copy
import json
import os
import subprocess
import sys

import pytest
import torch
from torch import nn

import stacr_b200 as S
from stacr_b200.composition import block_target_names, checkpoint_blocks, offload_blocks, saved_tensors_on_cpu, transformer_blocks
from stacr_b200.models import build_model
from stacr_b200.optim import AdamW, AdamW8bit
from stacr_b200.optim.adamw import (decode_first_moment, decode_second_moment, encode_first_moment, encode_second_moment)
from stacr_b200.training import configure_model, run_config, train_model, validate_config

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lm_batches(n, bs=4, seq=32, vocab=1024, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, vocab, (bs, seq), generator=g)
        out.append({"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()})
    return out


def test_validate_config_defaults_and_rejections():
    cfg = validate_config({})
    assert cfg["task"] == "synthetic" and cfg["method"] == "turbofast" and cfg["turbo_after_step"] == 50
    assert validate_config({"method": "stacr"})["turbo_after_step"] is None
    assert validate_config({"method": "stacr_checkpointing"})["checkpoint_every"] == 2
    for bad in ({"nope": 1}, {"method": "x"}, {"engine": "y"}, {"task": "language_modeling"}, {"steps": 0}, {"measure_from": 9, "steps": 5},
                {"method": "galore", "optimizer": "adamw"}):
        with pytest.raises(ValueError):
            validate_config(bad)


def test_synthetic_run_trains_and_reports():
    out = run_config({"task": "synthetic", "method": "turbofast", "steps": 6, "features": 64, "hidden": 32, "rank": 4, "device": "cpu",
                      "turbo_after_step": 3, "lr": 1e-2})
    assert out["wrapped_layers"] == 2 and out["steps_measured"] == 6 and out["wrapped_names"] == ["0", "2"]
    assert out["train_loss"] < out["first_loss"]


def test_tiny_gpt_language_model_loss_goes_down_with_stacr():
    torch.manual_seed(0)
    model = build_model("gpt-tiny", n_layer=2)
    batches = _lm_batches(2)
    out = train_model(model, batches, {"task": "language_modeling", "model_name": "gpt-tiny", "method": "stacr", "steps": 8, "lr": 3e-3,
                                       "device": "cpu", "rank": 4, "residual_budget": 0.01, "batch_size": 4, "seq_len": 32})
    assert out["wrapped_layers"] == 4 and out["tokens_per_second"] > 0
    assert out["train_loss"] < out["first_loss"]


def test_accumulation_matches_one_big_batch_for_the_baseline():
    torch.manual_seed(1)
    base = build_model("gpt-tiny", n_layer=1)
    big = _lm_batches(1, bs=4)
    halves = [{k: v[:2] for k, v in big[0].items()}, {k: v[2:] for k, v in big[0].items()}]
    m1, m2 = copy.deepcopy(base), copy.deepcopy(base)
    cfg = {"task": "language_modeling", "model_name": "gpt-tiny", "method": "baseline", "steps": 1, "lr": 1e-1, "device": "cpu",
           "optimizer": "stacr_b200.optim.factories:sgd"}
    train_model(m1, big, {**cfg, "batch_size": 4})
    train_model(m2, halves, {**cfg, "batch_size": 2, "gradient_accumulation_steps": 2})
    for a, b in zip(m1.parameters(), m2.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_nonfinite_loss_stops_before_the_update():
    class Bad(nn.Module):
        def __init__(self):
            super().__init__()
            self.w = nn.Parameter(torch.ones(1))

        def forward(self, **_):
            from types import SimpleNamespace
            return SimpleNamespace(loss=self.w.sum() * float("nan"))

    model = Bad()
    with pytest.raises(FloatingPointError):
        train_model(model, [{"inputs": torch.zeros(1)}], {"task": "synthetic", "method": "baseline", "steps": 1, "device": "cpu"})
    assert float(model.w) == 1.0


def test_checkpoint_complement_selection_and_composition_order():
    model = build_model("gpt-tiny", n_layer=4)
    layers, info = configure_model(model, {"task": "language_modeling", "model_name": "gpt-tiny", "method": "stacr_checkpointing",
                                           "checkpoint_every": 2, "offload_every": 2, "offload_offset": 1})
    assert info["checkpointed_blocks"] == [0, 2] and info["offloaded_blocks"] == [1, 3]
    assert all(".h.1." in n or ".h.3." in n for n in info["wrapped_names"]) and len(layers) == 4
    batch = _lm_batches(1)[0]
    model.train()
    S.set_step(layers, 0)
    model(**batch).loss.backward()
    assert all(p.grad is not None for p in model.parameters())
    blocks = transformer_blocks(model)
    with pytest.raises(ValueError):
        checkpoint_blocks(blocks, [0])
    with pytest.raises(ValueError):
        offload_blocks(blocks, [9])
    names = block_target_names(build_model("gpt-tiny", n_layer=2), transformer_blocks(build_model("gpt-tiny", n_layer=2)), lambda i: True)
    assert names == []  # different model object: no module identity in common


def test_offload_hook_preserves_values_and_strides():
    x = torch.randn(4, 6, 8).transpose(1, 2).requires_grad_(True)
    with saved_tensors_on_cpu(pin_memory=False):
        y = (x * x).sum()
    y.backward()
    torch.testing.assert_close(x.grad, 2 * x.detach())


def test_checkpoint_file_and_resume(tmp_path):
    path = tmp_path / "ckpt.pt"
    model = build_model("gpt-tiny", n_layer=1)
    cfg = {"task": "language_modeling", "model_name": "gpt-tiny", "method": "stacr", "steps": 2, "lr": 1e-3, "device": "cpu",
           "checkpoint_path": str(path)}
    train_model(model, _lm_batches(2), cfg)
    blob = torch.load(path, weights_only=False)
    assert {"model", "optimizer", "scaler", "step", "config", "rng_state", "cuda_rng_state"} <= set(blob)
    assert any(k.endswith("mlp.c_fc.basis") for k in blob["model"])
    fresh = build_model("gpt-tiny", n_layer=1)
    out = train_model(fresh, _lm_batches(2), {**cfg, "steps": 3, "resume_from": str(path), "checkpoint_path": None})
    assert out["steps_measured"] == 1


def test_8bit_codec_and_optimizer_on_cpu():
    torch.manual_seed(2)
    m = torch.randn(1000) * 1e-3
    codes, amax = encode_first_moment(m)
    back = decode_first_moment(codes, amax)
    assert codes.dtype == torch.uint8 and amax.numel() == 4
    per = amax.repeat_interleave(256)[:1000]
    # square-root companding: |dm| <= sqrt(|m| amax) / 127 (+ a half-step term near zero)
    assert ((back - m).abs() <= 1.01 * (m.abs() * per).sqrt() / 127 + per / 127 ** 2).all()
    v = torch.rand(1000) * 1e-6
    codes_v, amax_v = encode_second_moment(v)
    back_v = decode_second_moment(codes_v, amax_v)
    per_v = amax_v.repeat_interleave(256)[:1000]
    # fourth-root companding: |dv| <= (2 / 255) v^(3/4) amax^(1/4) (+ second-order terms)
    assert ((back_v - v).abs() <= 1.05 * (2 / 255) * v.pow(0.75) * per_v.pow(0.25) + 4 * per_v / 255 ** 2).all()
    w = nn.Parameter(torch.randn(80, 64))
    small = nn.Parameter(torch.randn(10))
    opt = AdamW8bit([w, small], lr=1e-2)
    w.grad, small.grad = torch.randn_like(w), torch.randn_like(small)
    opt.step()
    assert opt.state[w]["eight_bit"] and not opt.state[small]["eight_bit"]
    assert opt.state_bytes() < AdamW([nn.Parameter(torch.randn(80, 64))], lr=1e-2).state_bytes() + 2 * w.numel() * 4


def test_cli_dry_run_and_train(tmp_path):
    env = {**os.environ, "PYTHONPATH": REPO}
    dry = subprocess.run([sys.executable, "-m", "stacr", "train", "--config", "synthetic_stacr", "--dry-run", "--set", "rank=4",
                          "--set", "surface=on"], capture_output=True, text=True, env=env, cwd=REPO)
    assert dry.returncode == 0, dry.stderr
    cfg = json.loads(dry.stdout)
    assert cfg["rank"] == 4 and cfg["surface"] == "on"
    out = tmp_path / "r.csv"
    run = subprocess.run([sys.executable, "-m", "stacr", "train", "--config", "synthetic_stacr", "--steps", "3", "--device", "cpu",
                          "--output", str(out)], capture_output=True, text=True, env=env, cwd=REPO)
    assert run.returncode == 0, run.stderr
    assert out.exists() and out.with_suffix(".config.json").exists()
    bad = subprocess.run([sys.executable, "-m", "stacr", "train", "--config", "synthetic_stacr", "--set", "bogus=1"],
                         capture_output=True, text=True, env=env, cwd=REPO)
    assert bad.returncode != 0
    doc = subprocess.run([sys.executable, "-m", "stacr", "doctor"], capture_output=True, text=True, env=env, cwd=REPO)
    assert doc.returncode == 0 and "cuda_available" in doc.stdout


_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
import stacr_b200 as S
from stacr_b200.models import build_model
from stacr_b200.parallel import GradSync, broadcast_parameters, init_distributed
rank, world, _ = init_distributed("gloo")
torch.manual_seed(100 + rank)
model = build_model("gpt-tiny", n_layer=1)
broadcast_parameters(model)
layers = S.apply_stacr(model, rank=4, residual_budget=0.01, turbo_after_step=None)
sync = GradSync(model.parameters(), bucket_mb=0.05)
g = torch.Generator().manual_seed(7)
ids = torch.randint(0, 1024, (4, 32), generator=g)
mine = ids[rank * 2:(rank + 1) * 2]
S.set_step(layers, 0)
sync.zero_grad()
model(input_ids=mine, labels=mine).loss.backward()
sync.finish()
flat = sync.flat.clone()
gathered = [torch.zeros_like(flat) for _ in range(world)]
dist.all_gather(gathered, flat)
assert torch.equal(gathered[0], gathered[1]), "ranks disagree after reduction"
bases = [torch.zeros_like(layers[0].basis) for _ in range(world)]
dist.all_gather(bases, layers[0].basis.contiguous())
assert not torch.equal(bases[0], bases[1]), "bases must stay rank-local"
assert len(sync.buckets) > 1 and sync.reductions == len(sync.buckets)
if rank == 0:
    torch.save({"flat": flat, "names": [n for n, _ in model.named_parameters()]}, os.environ["OUT"])
dist.destroy_process_group()
'''


def test_two_rank_gloo_gradient_sync_matches_single_process_mean(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    out = tmp_path / "flat.pt"
    env = {**os.environ, "REPO": REPO, "OUT": str(out), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29611"}
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29611", str(script)], capture_output=True, text=True, env=env, timeout=240)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    got = torch.load(out)["flat"]
    # single-process oracle: uncompressed mean of the two shards' gradients has the same direction
    torch.manual_seed(100)
    model = build_model("gpt-tiny", n_layer=1)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 1024, (4, 32), generator=g)
    grads = []
    for r in range(2):
        model.zero_grad()
        part = ids[r * 2:(r + 1) * 2]
        model(input_ids=part, labels=part).loss.backward()
        grads.append(torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in model.parameters()]))
    want = (grads[0] + grads[1]) / 2
    # slots are padded to 4 elements: walk the same layout; parameters outside the compressed
    # layers must equal the mean of the two shards' gradients, compressed weights must agree in direction
    off = 0
    for (name, p), w in zip(model.named_parameters(), torch.split(want, [q.numel() for q in model.parameters()])):
        piece = got[off:off + p.numel()]
        off += (p.numel() + 3) // 4 * 4
        if name.endswith(("mlp.c_fc.weight", "mlp.c_proj.weight")):
            assert float(S.cosine_similarity(w, piece)) > 0.5, name
        else:
            torch.testing.assert_close(piece, w, rtol=1e-4, atol=1e-6, msg=name)


_FUSED_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
import stacr_b200 as S
from stacr_b200.models import build_model
from stacr_b200.parallel import GradSync, broadcast_parameters, init_distributed
rank, world, _ = init_distributed("gloo")
g = torch.Generator().manual_seed(7)
ids = torch.randint(0, 1024, (4, 32), generator=g)
mine = ids[rank * 2:(rank + 1) * 2]
results = []
for fused in (False, True):
    torch.manual_seed(5)
    model = build_model("gpt-tiny", n_layer=1, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    layers = S.apply_stacr(model, rank=4, residual_budget=0.01, turbo_after_step=None)
    sync = GradSync(model.parameters(), bucket_mb=0.05, fused=[l.weight for l in layers] if fused else ())
    assert sync.n_fused == (len(layers) if fused else 0)
    S.set_step(layers, 0)
    sync.zero_grad()
    with sync.no_sync():
        model(input_ids=mine, labels=mine).loss.backward()      # first micro-batch: nothing is reduced yet
    assert sync.reductions == 0
    model(input_ids=mine, labels=mine).loss.backward()
    sync.finish()
    results.append({n: p.grad.clone() for n, p in model.named_parameters()})
    sync.close()
for name, grad in results[0].items():
    torch.testing.assert_close(results[1][name], grad, rtol=1e-5, atol=1e-7, msg=name)
    other = [torch.zeros_like(grad) for _ in range(world)]
    dist.all_gather(other, results[1][name].contiguous())
    assert torch.equal(other[0], other[1]), name
print("FUSED_OK", flush=True)
dist.destroy_process_group()
'''


def test_two_rank_gloo_fused_parameter_slots_and_accumulation(tmp_path):
    script = tmp_path / "worker_fused.py"
    script.write_text(_FUSED_WORKER)
    env = {**os.environ, "REPO": REPO, "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29613"}
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29613", str(script)], capture_output=True, text=True, env=env, timeout=240)
    assert run.returncode == 0 and run.stdout.count("FUSED_OK") == 2, run.stdout[-2000:] + run.stderr[-2000:]


def test_grad_sync_and_its_buffer_are_collected_with_the_model():
    """The gradient hooks live in the tensors' C++ autograd state, out of the cycle collector's sight: they must not keep the
    sync object, its flat buffer and every parameter alive after the last outside reference is gone."""
    import gc
    import weakref

    import torch
    from torch import nn

    from stacr_b200.parallel.ddp import GradSync

    model = nn.Sequential(nn.Linear(16, 16), nn.Linear(16, 4))
    sync = GradSync(model.parameters(), backend="none")
    model(torch.randn(3, 16)).sum().backward()
    sync.finish()
    refs = [weakref.ref(model[0].weight), weakref.ref(sync), weakref.ref(sync.flat)]
    del model, sync
    gc.collect()
    assert all(r() is None for r in refs)


def test_gradient_slot_hand_over_counts_each_parameter_once():
    """A layer that wrote a parameter's gradient into its slot calls ``_sb_grad_ready`` and returns nothing to autograd."""
    import torch
    from torch import nn

    from stacr_b200.parallel.ddp import GradSync

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 4))
    sync = GradSync(model.parameters(), backend="none")
    w = model[0].weight
    assert callable(w._sb_grad_ready) and w._sb_grad_out.shape == w.shape
    sync.zero_grad()
    assert w.grad is None and w._sb_grad_fresh

    class Direct(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, weight):
            ctx.save_for_backward(x, weight)
            return x @ weight.t()

        @staticmethod
        def backward(ctx, dy):
            x, weight = ctx.saved_tensors
            slot = weight._sb_grad_out
            torch.mm(dy.t(), x, out=slot)
            weight._sb_grad_fresh = False
            weight._sb_grad_ready()
            return dy @ weight, None

    x = torch.randn(5, 8)
    y = model[1](torch.relu(Direct.apply(x, w) + model[0].bias))
    y.sum().backward()
    sync.finish()
    assert w.grad.data_ptr() == w._sb_grad_out.data_ptr()
    ref = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 4))
    ref.load_state_dict(model.state_dict())
    ref[1](torch.relu(ref[0](x))).sum().backward()
    for a, b in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-6)
    assert all(sync._written) and all(n == 0 for n in sync._pending)
    sync.close()
    assert not hasattr(w, "_sb_grad_ready")


_ZERO_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from stacr_b200.parallel import GradSync, ShardedGradSync
from stacr_b200.optim import AdamW
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
def build():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.GELU(), torch.nn.Linear(96, 4096 // 32), torch.nn.LayerNorm(128), torch.nn.Linear(128, 8))
def run(sharded, eight_bit):
    model = build()
    if sharded:
        sync = ShardedGradSync(model.parameters(), bucket_mb=0.02, shard_min_numel=2048)
        opt = AdamW(model.parameters(), lr=1e-2, weight_decay=0.01, eight_bit=eight_bit, min_8bit_size=1024, shard=sync)
    else:
        sync = GradSync(model.parameters(), bucket_mb=0.02)
        opt = AdamW(model.parameters(), lr=1e-2, weight_decay=0.01, eight_bit=eight_bit, min_8bit_size=1024)
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for step in range(6):
        x = torch.randn(16, 64, generator=g)
        sync.zero_grad()
        loss = model(x).square().mean()
        loss.backward()
        sync.finish()
        opt.step()
        losses.append(float(loss))
    if sharded:
        sync.gather_parameters()
        info = (sync.n_sharded, len(sync.buckets), [sync.owned_ranges(p) for p in model.parameters()])
    else:
        info = None
    return losses, [p.detach().clone() for p in model.parameters()], info
for eight in (False, True):
    la, pa, _ = run(False, eight)
    lb, pb, info = run(True, eight)
    worst = max(float((a - b).abs().max()) for a, b in zip(pa, pb))
    print(f"RANK{rank} eight_bit={eight} loss_diff={max(abs(a-b) for a,b in zip(la,lb)):.3e} param_diff={worst:.3e} sharded={info[0]} buckets={info[1]}", flush=True)
    if rank == 0 and not eight:
        print("RANGES", info[2], flush=True)
dist.destroy_process_group()
'''


def test_sharded_optimizer_over_two_gloo_ranks_reproduces_the_replicated_optimizer(tmp_path):
    """Reduce-to-owner + optimizer on the owned slices + publication of the update gives bit-identical parameters and losses to
    all-reduce + replicated optimizer, for fp32 and for 8-bit block-wise moments."""
    import os
    import subprocess
    import sys

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "zero_worker.py"
    script.write_text(_ZERO_WORKER)
    procs = []
    for rank in range(2):
        env = {**os.environ, "REPO": repo, "RANK": str(rank), "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29712"}
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for rank, out in enumerate(outs):
        lines = [l for l in out.splitlines() if l.startswith(f"RANK{rank} ")]
        assert len(lines) == 2, out[-2000:]
        for line in lines:
            assert "loss_diff=0.000e+00" in line and "param_diff=0.000e+00" in line and "sharded=2" in line, line
    assert "RANGES [[(0, 4096)]" in outs[0]      # rank 0 updates the first two of the three chunks of the first matrix
