"""Data-parallel grid: per-rank peak memory and throughput of baseline / STAC-R / Turbo-fast / checkpoint compositions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m experiments.benchmarks.distributed_data
    python -m experiments.benchmarks.distributed_data --smoke      # one CPU rank over gloo, tiny model, 3 steps
    python -m experiments.benchmarks.distributed_data --dry-run    # print the cell plan; also: --seeds 42,123 --steps N --output FILE

Gradients are averaged by ``stacr_b200.parallel.GradSync`` (flat buffer, bucketed, overlapped with backward; NVLink
all-reduce kernels when symmetric memory is available, else NCCL/gloo); bases stay rank-local.
Parity: experiments/benchmarks/distributed_data.py:1-217 of the reference project (seven arms, three seeds,
strided batch split, per-rank peak gather, OOM/error rows).
"""

from __future__ import annotations

import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

import stacr_b200 as S
from stacr_b200.parallel import GradSync, broadcast_parameters, init_distributed

from . import common
from .registry import EXPERIMENTS

SEEDS = [42, 123, 456]


def complement(k: int):
    """Predicate selecting the blocks a 1-in-``k`` checkpointing plan leaves alone (``index % k != 0``)."""
    return lambda index, _k=int(k): index % _k != 0


def one_run(cell: dict, seed: int, *, device: str, smoke: bool = False) -> dict:
    cell = dict(cell)
    method = cell.pop("method")
    steps, measure_from = (4, 1) if smoke else (cell.pop("steps", 120), cell.pop("measure_from", 20))
    model_id, bs, seq = ("gpt-tiny", 2, 64) if smoke else (cell["model_id"], cell["bs"], cell["seq"])
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    common.free_all()
    common.set_seed(seed)
    model = common.load_model(model_id, device)
    broadcast_parameters(model)
    n_ckpt = common.apply_selective_checkpointing(model, cell.get("ckpt_every", 0))
    layers = []
    if cell.get("stacr_cfg"):
        k = cell.get("complement")
        cfg = dict(cell["stacr_cfg"], min_features=64) if smoke else cell["stacr_cfg"]
        layers = common.stacr_on_blocks(model, cfg, complement(k) if k else None)
    opt = common.build_optimizer(model, 5e-5, device == "cuda")
    sync = GradSync(model.parameters()) if world > 1 else None
    vocab = model.config.vocab_size
    batches = common.get_batches(model_id, "train", bs, seq, steps * world, "synthetic", device, vocab, seed)[rank::world][:steps]
    ev = None
    t0 = None
    loss = None
    for i, batch in enumerate(batches):
        S.set_step(layers, i)
        if i == measure_from:
            common.sync()
            if device == "cuda":
                torch.cuda.reset_peak_memory_stats()
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
            t0 = time.perf_counter()
        sync.zero_grad() if sync else opt.zero_grad(set_to_none=True)
        with common.amp_ctx(device == "cuda"):
            loss = model(**batch).loss
        loss.backward()
        if sync:
            sync.finish()
        opt.step()
    if ev:
        ev[1].record()
        common.sync()
        dt = ev[0].elapsed_time(ev[1]) / 1e3
    else:
        dt = time.perf_counter() - (t0 or time.perf_counter())
    peak = torch.cuda.max_memory_allocated() if device == "cuda" else 0
    peaks = [float(peak)]
    if world > 1:
        buf = [torch.zeros(1, dtype=torch.float64, device=device) for _ in range(world)]
        dist.all_gather(buf, torch.tensor([float(peak)], dtype=torch.float64, device=device))
        peaks = [float(b) for b in buf]
    measured = max(0, len(batches) - measure_from)
    final_loss = float(loss.detach())
    # the symmetric-memory gradient buffer is mapped outside the caching allocator, so the allocator's peak does not hold it
    outside = sync.flat.numel() * sync.flat.element_size() if sync and sync.backend == "symm" else 0
    if sync:
        sync.close()         # unhook before the next arm builds its own model and buffer
    return {"tag": f"ddp_w{world}", "method": method, "seed": seed, "world_size": world, "model": model_id, "bs_per_rank": bs, "seq": seq,
            "steps": steps, "steps_measured": measured, "n_checkpointed_blocks": n_ckpt, "n_wrapped_layers": len(layers), "time_s": dt,
            "peak_bytes": peak, "peak_GiB": common.gib(peak), "grad_buffer_outside_allocator_GiB": common.gib(outside), "peak_GiB_all_ranks": [common.gib(p) for p in peaks],
            "tokens_per_s_per_rank": bs * seq * measured / dt if dt > 0 and measured else None, "final_train_loss": final_loss,
            "comm": sync.backend if sync else "none", "status": "ok"}


def _flag(name: str, default: str) -> str:
    """Value of ``name VALUE`` or ``name=VALUE`` on the command line."""
    for i, arg in enumerate(sys.argv):
        if arg == name and i + 1 < len(sys.argv):
            return sys.argv[i + 1]
        if arg.startswith(name + "="):
            return arg.split("=", 1)[1]
    return default


def main() -> int:
    smoke = "--smoke" in sys.argv
    cells = EXPERIMENTS["distributed_data"]["cells"]
    only = os.environ.get("STACR_ARM", "").strip()
    skip = set(os.environ.get("STACR_SKIP_ARMS", "").replace(",", " ").split())
    cells = [c for c in cells if (not only or c["method"] == only) and c["method"] not in skip]
    if not cells:
        raise SystemExit("STACR_ARM / STACR_SKIP_ARMS removed every arm")
    seeds = [int(x) for x in _flag("--seeds", "").replace(",", " ").split()] or SEEDS
    steps = _flag("--steps", "")
    if steps:
        cells = [dict(c, steps=int(steps), measure_from=min(c.get("measure_from", 20), max(1, int(steps) // 4))) for c in cells]
    if "--dry-run" in sys.argv:
        import json
        print(json.dumps({"experiment": "distributed_data", "n_cells": len(cells) * len(seeds), "seeds": seeds, "cells": cells}, indent=1))
        return 0
    if smoke:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        dist.init_process_group("gloo", rank=0, world_size=1)
        for cell in cells:
            rec = one_run(cell, 42, device="cpu", smoke=True)
            print(f"  smoke {cell['method']:22s} ok wrapped={rec['n_wrapped_layers']} ckpt={rec['n_checkpointed_blocks']} loss={rec['final_train_loss']:.4f}", flush=True)
        dist.destroy_process_group()
        return 0
    rank, world, local = init_distributed("nccl")
    out = Path(_flag("--output", "") or common.RESULTS / "x7_ddp.jsonl")
    for cell in cells:
        for seed in seeds:
            try:
                rec = one_run(cell, seed, device="cuda")
            except torch.cuda.OutOfMemoryError:
                rec = {"tag": f"ddp_w{world}", "method": cell["method"], "seed": seed, "status": "OOM"}
                torch.cuda.empty_cache()
            except Exception as exc:  # noqa: BLE001
                rec = {"tag": f"ddp_w{world}", "method": cell["method"], "seed": seed, "status": "error", "error": f"{type(exc).__name__}: {str(exc)[:200]}"}
                torch.cuda.empty_cache()
            if rank == 0:
                common.emit(rec, out)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
