"""The non-headline benchmark configurations run through the UNMODIFIED reference package.

    python experiments/benchmarks/reference_arms.py --config gpt2m_turbo_dp --steps 10
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 experiments/benchmarks/reference_arms.py --config gpt2l_tp
    python experiments/benchmarks/reference_arms.py --config bert_adaptive_composed

The counterpart of ``baseline_configs.py`` for the reference arm: the same three configurations, same shapes, same
synthetic data and random initialisation, but every model is a Hugging Face model built from a config and every
compression / parallelism call is the reference's own (``apply_stacr``, ``stacr.protocols.tp_gpt2``,
``stacr.training.configure_model``), imported from the offline install under ``baseline/_ref``.  Nothing of this
repository's package is imported: the file is run by path, and the repository root is taken off ``sys.path`` because
the reference package has the same top-level name as this repository's alias package.

Prints one JSON line per timed phase with ``"impl": "reference"``; when the reference cannot run a configuration on this
image the line is ``{"impl": "reference", "config": ..., "unavailable": "<why>"}`` and the exit code is 0.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF_ROOT = os.path.join(REPO, "baseline", "_ref")


def _emit(rank, **row):
    if rank == 0:
        print(json.dumps({"impl": "reference", **row}), flush=True)


def _timed(torch, dist, steps, fn, world) -> float:
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / 1e3], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _tokens(torch, vocab, batch, seq, count, seed, device):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (batch, seq), generator=gen).to(device) for _ in range(count)]


def run_gpt2m_turbo_dp(args, ref, torch, dist, rank, world, dev):
    from torch.nn.parallel import DistributedDataParallel as DDP
    from transformers import GPT2Config, GPT2LMHeadModel

    batch, seq = 8, 1024
    torch.manual_seed(1234)
    cfg = GPT2Config(n_embd=1024, n_layer=24, n_head=16, n_positions=1024, vocab_size=50257, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    model = GPT2LMHeadModel(cfg).to(dev).train()
    layers = ref.apply_stacr(model, rank=8, residual_budget=0.005, turbo_after_step=50, surface="mlp")
    net = DDP(model, device_ids=[dev.index], static_graph=True, broadcast_buffers=False) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=5e-5, weight_decay=0.0)
    data = _tokens(torch, cfg.vocab_size, batch, seq, 8, 100 + rank, dev)
    state = {"step": 0}

    def step(_i):
        ref.set_step(layers, state["step"])
        ids = data[state["step"] % len(data)]
        state["step"] += 1
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            net(input_ids=ids, labels=ids).loss.backward()
        opt.step()

    for phase, until in (("full (steps < 50)", 5), ("turbo (steps >= 50)", 55)):
        while state["step"] < until:
            step(0)
        torch.cuda.reset_peak_memory_stats(dev)
        secs = _timed(torch, dist, args.steps, step, world)
        rows = batch * seq
        _emit(rank, config="gpt2m_turbo_dp", phase=phase, n_gpus=world, steps=args.steps, tokens_per_second=world * rows * args.steps / secs,
              ms_per_step=1e3 * secs / args.steps, peak_allocated_gb=torch.cuda.max_memory_allocated(dev) / 1e9, wrapped_layers=len(layers),
              optimizer="torch.optim.AdamW", model="HF GPT2LMHeadModel from config", first_step_in_phase=until)


def run_gpt2l_tp(args, ref, torch, dist, rank, world, dev):
    from stacr.protocols.tensor_parallel import sync_replicated_grads
    from stacr.protocols.tp_gpt2 import apply_tensor_parallel_gpt2, disable_tp_dropout, get_tp_stacr_targets
    from transformers import GPT2Config, GPT2LMHeadModel

    batch, seq = 4, 1024
    torch.manual_seed(7)
    cfg = GPT2Config(n_embd=1280, n_layer=36, n_head=20, n_positions=1024, vocab_size=50257, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    model = GPT2LMHeadModel(cfg).to(dev).train()
    scope = "full" if cfg.n_head % world == 0 else "mlp_only"      # 20 heads: degree 8 shards the MLPs only
    if world > 1:
        apply_tensor_parallel_gpt2(model, rank, world, None, scope=scope)
        disable_tp_dropout(model)
        names = get_tp_stacr_targets(model, "all_linear")
        layers = ref.apply_stacr(model, surface="none", target_names=names, rank=8, residual_budget=0.005, residual_mode="block_sparse",
                                 turbo_after_step=None)
    else:
        layers = ref.apply_stacr(model, surface="mlp+attention", rank=8, residual_budget=0.005, residual_mode="block_sparse", turbo_after_step=None)
    opt = torch.optim.AdamW(model.parameters(), lr=5e-5, weight_decay=0.0)
    data = _tokens(torch, cfg.vocab_size, batch, seq, 8, 100, dev)
    state = {"step": 0}

    def step(_i):
        ref.set_step(layers, state["step"])
        ids = data[state["step"] % len(data)]
        state["step"] += 1
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            model(input_ids=ids, labels=ids).loss.backward()
        if world > 1:
            sync_replicated_grads(model, None)
        opt.step()

    for _ in range(max(3, args.warmup)):
        step(0)
    torch.cuda.reset_peak_memory_stats(dev)
    secs = _timed(torch, dist, args.steps, step, world)
    _emit(rank, config="gpt2l_tp", tp_degree=world, tp_scope=scope if world > 1 else "none", steps=args.steps, tokens_per_second=batch * seq * args.steps / secs, ms_per_step=1e3 * secs / args.steps,
          peak_allocated_gb=torch.cuda.max_memory_allocated(dev) / 1e9, wrapped_layers=len(layers), optimizer="torch.optim.AdamW",
          model="HF GPT2LMHeadModel from config; the reference's own tp_gpt2 module replacement and sync_replicated_grads")


def run_bert_adaptive_composed(args, ref, torch, dist, rank, world, dev):
    """bf16 autocast as configured; if the reference's adaptive engine cannot run in bf16 on this torch (its sparse residual
    product has no bf16 CUDA kernel), the same configuration is timed in fp32 and the line says so."""
    try:
        _bert_adaptive_composed(args, ref, torch, dist, rank, world, dev, "bf16")
    except (NotImplementedError, RuntimeError) as exc:
        _emit(rank, config="bert_adaptive_composed", amp="bf16", unavailable=f"{type(exc).__name__}: {str(exc)[:200]}")
        torch.cuda.empty_cache()
        _bert_adaptive_composed(args, ref, torch, dist, rank, world, dev, "fp32")


def _bert_adaptive_composed(args, ref, torch, dist, rank, world, dev, amp):
    import contextlib

    from stacr.training import configure_model
    from torch.nn.parallel import DistributedDataParallel as DDP
    from transformers import BertConfig, BertForSequenceClassification

    batch, seq = 32, 128
    torch.manual_seed(1234)
    cfg = BertConfig(hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, num_labels=2)
    model = BertForSequenceClassification(cfg).to(dev).train()
    run_cfg = {
        "task": "sequence_classification", "method": "stacr_checkpointing", "engine": "adaptive", "model_name": "bert-base-uncased",
        "seq_len": seq, "batch_size": batch, "steps": 100, "lr": 2.0e-5, "amp": amp if amp == "bf16" else "none", "rank": 32, "residual_budget": 0.005,
        "checkpoint_every": 2, "offload_every": 2, "offload_offset": 1,
        "compression": {"quantize_coefficients": True, "rank_mode": "sensitivity", "rank_min": 4, "rank_max": 32, "refresh_trigger": "residual_energy",
                        "residual_mode": "topk"},
    }
    layers, info = configure_model(model, run_cfg)
    net = DDP(model, device_ids=[dev.index], broadcast_buffers=False) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=2e-5, weight_decay=0.0)
    gen = torch.Generator().manual_seed(100 + rank)
    data = [(torch.randint(0, cfg.vocab_size, (batch, seq), generator=gen).to(dev), torch.bernoulli(torch.full((batch,), 0.5), generator=gen).long().to(dev))
            for _ in range(8)]
    state = {"step": 0}

    def step(_i):
        ref.set_step(layers, state["step"])
        ids, labels = data[state["step"] % len(data)]
        state["step"] += 1
        opt.zero_grad(set_to_none=True)
        with (torch.autocast("cuda", dtype=torch.bfloat16) if amp == "bf16" else contextlib.nullcontext()):
            net(input_ids=ids, attention_mask=torch.ones_like(ids), labels=labels).loss.backward()
        opt.step()

    for _ in range(max(3, args.warmup)):
        step(0)
    torch.cuda.reset_peak_memory_stats(dev)
    secs = _timed(torch, dist, args.steps, step, world)
    _emit(rank, config="bert_adaptive_composed", amp=amp, n_gpus=world, steps=args.steps, tokens_per_second=world * batch * seq * args.steps / secs,
          ms_per_step=1e3 * secs / args.steps, peak_allocated_gb=torch.cuda.max_memory_allocated(dev) / 1e9, wrapped_layers=len(layers),
          checkpointed_blocks=info["checkpointed_blocks"], offloaded_blocks=info["offloaded_blocks"], optimizer="torch.optim.AdamW",
          model="HF BertForSequenceClassification from config; the reference's own configure_model (adaptive engine, checkpoint + offload)")


RUNNERS = {"gpt2m_turbo_dp": run_gpt2m_turbo_dp, "gpt2l_tp": run_gpt2l_tp, "bert_adaptive_composed": run_bert_adaptive_composed}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--config", required=True, choices=sorted(RUNNERS))
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=5)
    args = parser.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    if not os.path.isdir(os.path.join(REF_ROOT, "stacr")):
        _emit(rank, config=args.config, unavailable="baseline/_ref is missing (offline pip install of the reference not present)")
        return 0
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") not in (REPO, HERE)]
    sys.path.insert(0, REF_ROOT)
    if os.environ.get("NCCL_DEBUG", "VERSION") == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    try:
        import stacr as ref
        import torch
        import torch.distributed as dist

        assert os.path.abspath(ref.__file__).startswith(REF_ROOT), ref.__file__
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=dev)
        RUNNERS[args.config](args, ref, torch, dist, rank, world, dev)
        torch.cuda.synchronize()
        if world > 1:
            dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001 - the reference on a newer transformers / without its optional libraries
        import traceback

        traceback.print_exc(file=sys.stderr)
        _emit(rank, config=args.config, unavailable=f"{type(exc).__name__}: {str(exc)[:300]}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
