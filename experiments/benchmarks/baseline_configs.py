"""The benchmark configurations other than the headline one, through this framework's public API.

    python -m experiments.benchmarks.baseline_configs --config gpt2m_turbo_dp --steps 10
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m experiments.benchmarks.baseline_configs --config gpt2l_tp
    python -m experiments.benchmarks.baseline_configs --config bert_adaptive_composed

* ``gpt2m_turbo_dp``: GPT-2 medium (24 x 1024, seq 1024, batch 8 per GPU), Turbo-fast STAC-R on the MLP surface
  (rank 8, budget 0.005, turbo_after_step 50), data parallel.  Timed twice: in the full phase (before step 50) and in the
  turbo phase (after it).
* ``gpt2l_tp``: GPT-2 large (36 x 1280, seq 1024, batch 4), tensor parallel over all ranks with column-parallel up/QKV and
  row-parallel down/out projections, all four compressed (rank 8, block-sparse residual, budget 0.005).
* ``bert_adaptive_composed``: BERT-base classifier (seq 128, batch 32 per GPU), adaptive engine with int8 coefficients,
  rank 4-32, residual-triggered refresh, every other block checkpointed and the rest offloaded; data parallel.

Each run prints one JSON line per timed phase: tokens/s over all ranks (CUDA events, max over ranks, after warm-up), peak
allocated memory and the bytes the wrapped layers keep for backward.  Weights are random and tokens synthetic.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _timed(steps, fn, world) -> float:
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


def _tokens(vocab, batch, seq, count, seed, device):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (batch, seq), generator=gen).to(device) for _ in range(count)]


def _reports(args, step, rank) -> None:
    """Optional per-kernel device times and idle-gap report of two more steps (the benchmark's own profiler helpers)."""
    if not (args.kernel_table or args.gap_report):
        return
    import importlib.util
    import pathlib

    spec = importlib.util.spec_from_file_location("_bench", pathlib.Path(__file__).resolve().parents[2] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    if args.kernel_table:
        bench.kernel_table(torch, step, args.kernel_table if rank == 0 else os.devnull)
    if args.gap_report:
        bench.gap_report(torch, step, args.gap_report if rank == 0 else os.devnull)


def _emit(rank, **row):
    if rank == 0:
        print(json.dumps(row), flush=True)


def run_gpt2m_turbo_dp(args, rank, world, dev):
    import stacr_b200 as S
    from stacr_b200.models import build_model
    from stacr_b200.optim import AdamW
    from stacr_b200.parallel import GradSync, broadcast_parameters

    batch, seq = 8, 1024
    model = build_model("gpt2-medium").to(dev).train()
    broadcast_parameters(model)
    layers = S.apply_stacr(model, rank=8, residual_budget=0.005, turbo_after_step=50, surface="mlp")
    opt = AdamW(model.parameters(), lr=5e-5, weight_decay=0.0, bf16_shadow=True)
    sync = GradSync(model.parameters()) if world > 1 else None
    data = _tokens(model.config.vocab_size, batch, seq, 8, 100 + rank, dev)
    state = {"step": 0}

    def core(ids):
        sync.zero_grad() if sync else opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        if sync:
            sync.finish()
        opt.step()
        return loss

    def eager(_i):
        S.set_step(layers, state["step"])
        ids = data[state["step"] % len(data)]
        state["step"] += 1
        core(ids)

    use_graph = args.graph == "on" and (sync is None or sync.backend == "symm")
    for phase, until in (("full (steps < 50)", 5), ("turbo (steps >= 50)", 55)):
        while state["step"] < until:
            eager(0)
        step = eager
        if use_graph:      # one graph per phase: the kernels of a step change when the residual is dropped at step 50
            from stacr_b200.graphs import GraphedStep

            graphed = GraphedStep(core, [data[0]], optimizer=opt, layers=layers, first_step=state["step"], warmup=2)
            state["step"] = graphed.step

            def step(_i, graphed=graphed):
                graphed(data[graphed.step % len(data)])
                state["step"] = graphed.step
        torch.cuda.reset_peak_memory_stats(dev)
        secs = _timed(args.steps, step, world)
        rows = batch * seq
        _emit(rank, config="gpt2m_turbo_dp", phase=phase, n_gpus=world, steps=args.steps, tokens_per_second=world * rows * args.steps / secs,
              ms_per_step=1e3 * secs / args.steps, peak_allocated_gb=torch.cuda.max_memory_allocated(dev) / 1e9,
              saved_gb_wrapped=sum(l.stored_bytes(rows, 2)["total"] for l in layers) / 1e9, dense_gb_same_layers=sum(rows * l.in_features * 2 for l in layers) / 1e9,
              first_step_in_phase=until, cuda_graph=use_graph)


def run_gpt2l_tp(args, rank, world, dev):
    import stacr_b200 as S
    from stacr_b200.models import build_model
    from stacr_b200.optim import AdamW
    from stacr_b200.parallel import GradSync
    from stacr_b200.protocols.tensor_parallel import replicated_parameters
    from stacr_b200.protocols.tp_gpt2 import apply_tensor_parallel_gpt2, disable_tp_dropout, get_tp_stacr_targets

    batch, seq = 4, 1024
    torch.manual_seed(7)                                   # every rank builds the same full model, then keeps its shard
    model = build_model("gpt2-large").to(dev).train()
    # GPT-2 large has 20 heads: degrees that do not divide them (8) shard the MLPs only and keep attention replicated
    scope = "full" if model.config.n_head % world == 0 else "mlp_only"
    apply_tensor_parallel_gpt2(model, rank, world, None, scope=scope)
    disable_tp_dropout(model)
    names = get_tp_stacr_targets(model, "all_linear")
    layers = S.apply_stacr(model, surface="none", target_names=names, rank=8, residual_budget=0.005, residual_mode="block_sparse",
                           turbo_after_step=None, allow_empty=False)
    opt = AdamW(model.parameters(), lr=5e-5, weight_decay=0.0, bf16_shadow=True)
    # gradients of the replicated parameters (embeddings, LayerNorms) are averaged over the ranks in one flat symmetric buffer by
    # the in-tree all-reduce, overlapped with backward; the shards' gradients are local
    sync = GradSync([p for _, p in replicated_parameters(model)]) if world > 1 else None
    data = _tokens(model.config.vocab_size, batch, seq, 8, 100, dev)   # the same batch on every rank: this is model parallelism
    state = {"step": 0}

    def core(ids):
        opt.zero_grad(set_to_none=True)
        if sync:
            sync.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        if sync:
            sync.finish()
        opt.step()
        return loss

    def step(_i):
        S.set_step(layers, state["step"])
        ids = data[state["step"] % len(data)]
        state["step"] += 1
        core(ids)

    for _ in range(max(3, args.warmup)):
        step(0)
    use_graph = args.graph == "on" and (sync is None or sync.backend == "symm")
    if use_graph:
        from stacr_b200.graphs import GraphedStep

        graphed = GraphedStep(core, [data[0]], optimizer=opt, layers=layers, first_step=state["step"], warmup=2)

        def step(_i):  # noqa: F811 - the replayed form of the step above
            graphed(data[graphed.step % len(data)])
    torch.cuda.reset_peak_memory_stats(dev)
    secs = _timed(args.steps, step, world)
    _reports(args, step, rank)
    _emit(rank, config="gpt2l_tp", tp_degree=world, tp_scope=scope, steps=args.steps, tokens_per_second=batch * seq * args.steps / secs, ms_per_step=1e3 * secs / args.steps,
          peak_allocated_gb=torch.cuda.max_memory_allocated(dev) / 1e9, wrapped_layers=len(layers), cuda_graph=use_graph,
          saved_gb_wrapped=sum(l.stored_bytes(batch * seq, 2)["total"] for l in layers) / 1e9,
          dense_gb_same_layers=sum(batch * seq * l.in_features * 2 for l in layers) / 1e9)


def run_bert_adaptive_composed(args, rank, world, dev):
    from stacr_b200.adaptive import set_stacr_runtime_state
    from stacr_b200.models import build_model
    from stacr_b200.optim import AdamW
    from stacr_b200.parallel import GradSync, broadcast_parameters
    from stacr_b200.training import configure_model
    from stacr_b200.utils import load_yaml
    from stacr_b200.cli import resolve_config

    cfg = load_yaml(resolve_config("bert_adaptive_composed"))
    batch, seq = int(cfg["batch_size"]), int(cfg["seq_len"])
    model = build_model(cfg["model_name"], "sequence_classification").to(dev).train()
    broadcast_parameters(model)
    layers, info = configure_model(model, cfg)
    opt = AdamW(model.parameters(), lr=float(cfg["lr"]), weight_decay=0.0, bf16_shadow=True)
    sync = GradSync(model.parameters()) if world > 1 else None
    gen = torch.Generator().manual_seed(100 + rank)
    data = [(torch.randint(0, model.config.vocab_size, (batch, seq), generator=gen).to(dev), torch.bernoulli(torch.full((batch,), 0.5), generator=gen).long().to(dev))
            for _ in range(8)]
    state = {"step": 0}

    def step(_i):
        set_stacr_runtime_state(model, state["step"], 0, 1, 10_000)
        ids, labels = data[state["step"] % len(data)]
        state["step"] += 1
        sync.zero_grad() if sync else opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            model(input_ids=ids, attention_mask=torch.ones_like(ids), labels=labels).loss.backward()
        if sync:
            sync.finish()
        opt.step()

    for _ in range(max(3, args.warmup)):
        step(0)
    torch.cuda.reset_peak_memory_stats(dev)
    secs = _timed(args.steps, step, world)
    _emit(rank, config="bert_adaptive_composed", n_gpus=world, steps=args.steps, tokens_per_second=world * batch * seq * args.steps / secs,
          ms_per_step=1e3 * secs / args.steps, peak_allocated_gb=torch.cuda.max_memory_allocated(dev) / 1e9, wrapped_layers=len(layers),
          checkpointed_blocks=info["checkpointed_blocks"], offloaded_blocks=info["offloaded_blocks"],
          active_ranks=sorted({int(l.layer_state["active_rank"]) for l in layers}))


RUNNERS = {"gpt2m_turbo_dp": run_gpt2m_turbo_dp, "gpt2l_tp": run_gpt2l_tp, "bert_adaptive_composed": run_bert_adaptive_composed}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--config", required=True, choices=sorted(RUNNERS))
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--graph", default="on", choices=["on", "off"], help="replay the training step from a CUDA graph (projection-engine configurations)")
    parser.add_argument("--kernel-table", metavar="FILE", help="gpt2l_tp: write per-kernel device times of two more steps to FILE")
    parser.add_argument("--gap-report", metavar="FILE", help="gpt2l_tp: write where the GPU idles inside two more steps to FILE")
    args = parser.parse_args(argv)
    from stacr_b200.ops import _lib
    from stacr_b200.parallel import init_distributed

    if os.environ.get("NCCL_DEBUG", "VERSION") == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    rank, world, local = init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    RUNNERS[args.config](args, rank, world, dev)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
