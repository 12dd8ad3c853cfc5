"""Sharded data parallel (FSDP2 ``fully_shard`` per block, then the root) with STAC-R applied before sharding.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m experiments.benchmarks.distributed_sharding
    python -m experiments.benchmarks.distributed_sharding --smoke      # one rank, tiny model
    python -m experiments.benchmarks.distributed_sharding --dry-run    # the cell plan; also: --models a,b --steps N --output FILE

Parity: experiments/benchmarks/distributed_sharding.py:1-362 of the reference project (bf16 parameters, torch AdamW,
per-rank peak via all_reduce MAX, cohorts up to 14B parameters).  Compression state stays per rank; the sharded
parameters are all-gathered by FSDP2 before the compressed layer's kernels see them.
"""

from __future__ import annotations

import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

import stacr_b200 as S
from stacr_b200.composition import transformer_blocks

from . import common
from .registry import EXPERIMENTS


def complement(k: int):
    """Predicate selecting the blocks a 1-in-``k`` checkpointing plan leaves alone (``index % k != 0``)."""
    return lambda index, _k=int(k): index % _k != 0


def arm_filter(arms):
    """Restrict a cohort's arms by environment: ``STACR_ARM`` keeps one method, ``STACR_SKIP_ARMS`` drops a list.

    ``arms`` is a list of cells (mappings with a ``method`` key) or of ``(name, options)`` pairs.
    """
    def name_of(arm):
        return arm["method"] if isinstance(arm, dict) else arm[0]

    only = os.environ.get("STACR_ARM", "").strip()
    skip = set(os.environ.get("STACR_SKIP_ARMS", "").replace(",", " ").split())
    kept = [a for a in arms if name_of(a) not in skip]
    if only:
        kept = [a for a in kept if name_of(a) == only]
        if not kept:
            raise SystemExit(f"STACR_ARM={only!r} matches no arm in this cohort")
    return kept


def build_opt_honest(model, lr: float = 5e-5):
    """Plain torch AdamW whose moments take the parameters' dtype; returns ``(optimizer, label, state_dtype)``.

    Sharded parameters are DTensors, which the in-tree multi-tensor AdamW does not take, so the sharded cohorts
    report the optimizer they really ran.
    """
    dtype = next(model.parameters()).dtype
    short = str(dtype).replace("torch.", "")
    return torch.optim.AdamW(model.parameters(), lr=lr), f"torch_adamw_{short}_states", str(dtype)


def shard(model):
    """FSDP2: shard every transformer block, then the root module."""
    from torch.distributed.fsdp import fully_shard

    for block in transformer_blocks(model):
        fully_shard(block)
    fully_shard(model)
    return model


def one_run(cell: dict, seed: int, smoke: bool = False) -> dict:
    cell = dict(cell)
    method = cell.pop("method")
    model_id, bs, seq = ("llama-tiny", 2, 64) if smoke else (cell["model_id"], cell["bs"], cell["seq"])
    steps, measure_from = (4, 1) if smoke else (int(cell.get("steps", 30)), int(cell.get("measure_from", 10)))
    device = "cuda" if torch.cuda.is_available() else "cpu"
    common.free_all()
    common.set_seed(seed)
    model = common.load_model(model_id, device, dtype=torch.bfloat16 if device == "cuda" else torch.float32)
    layers = common.stacr_on_blocks(model, dict(cell["stacr_cfg"], min_features=64 if smoke else 256)) if cell.get("stacr_cfg") else []
    ckpt_every = int(cell.get("ckpt_every", 0) or 0)
    n_ckpt = common.apply_selective_checkpointing(model, ckpt_every) if ckpt_every else 0
    shard(model)
    opt, opt_label, state_dtype = build_opt_honest(model)
    vocab = model.config.vocab_size
    rank, world = dist.get_rank(), dist.get_world_size()
    batches = common.get_batches(model_id, "train", bs, seq, steps * world, "synthetic", device, vocab, seed)[rank::world][:steps]
    t0, loss = None, None
    for i, batch in enumerate(batches):
        S.set_step(layers, i)
        if i == measure_from:
            common.sync()
            if device == "cuda":
                torch.cuda.reset_peak_memory_stats()
            t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        loss = model(**batch).loss
        loss.backward()
        opt.step()
    common.sync()
    dt = time.perf_counter() - (t0 or time.perf_counter())
    peak = torch.tensor([float(torch.cuda.max_memory_allocated() if device == "cuda" else 0)], device=device)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    measured = max(0, len(batches) - measure_from)
    return {"tag": f"fsdp2_w{world}", "method": method, "seed": seed, "world_size": world, "model": model_id, "bs_per_rank": bs, "seq": seq,
            "n_wrapped_layers": len(layers), "n_checkpointed_blocks": n_ckpt, "optimizer_actual": opt_label, "optimizer_state_dtype": state_dtype, "time_s": dt, "peak_GiB_max_rank": common.gib(float(peak)),
            "tokens_per_s_per_rank": bs * seq * measured / dt if dt > 0 and measured else None, "final_train_loss": float(loss.detach()), "status": "ok"}


def run_cohort(name: str, cells, out, smoke: bool = False, seeds=(42,)) -> list:
    """Run every arm of one cohort for every seed; rank 0 appends a record per run (``OOM``/``error`` runs included)."""
    rank, world = dist.get_rank(), dist.get_world_size()
    records, base = [], None
    for cell in arm_filter(cells):
        for seed in seeds:
            try:
                rec = one_run(cell, seed, smoke=smoke)
            except torch.cuda.OutOfMemoryError:
                rec = {"tag": f"fsdp2_w{world}", "method": cell["method"], "model": cell.get("model_id"), "seed": seed, "status": "OOM"}
                torch.cuda.empty_cache()
            except Exception as exc:  # a failed arm must not take the cohort down with it
                rec = {"tag": f"fsdp2_w{world}", "method": cell["method"], "model": cell.get("model_id"), "seed": seed, "status": "error",
                       "error": f"{type(exc).__name__}: {str(exc)[:200]}"}
                if torch.cuda.is_available():
                    torch.cuda.empty_cache()
            rec["cohort"] = name
            if rec.get("status") == "ok" and cell["method"] == "baseline" and base is None:
                base = rec["peak_GiB_max_rank"]
            if base and rec.get("status") == "ok":
                rec["peak_saving_pct_vs_baseline"] = 100.0 * (base - rec["peak_GiB_max_rank"]) / base
            records.append(rec)
            if rank == 0:
                if smoke:
                    print(f"  smoke {rec['method']:14s} {rec.get('status')} loss={rec.get('final_train_loss')}", flush=True)
                else:
                    common.emit(rec, out)
    return records


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
    cells = EXPERIMENTS["distributed_sharding"]["cells"]
    wanted = set(_flag("--models", "").replace(",", " ").split())
    if wanted:
        cells = [c for c in cells if c.get("model_id") in wanted]
    if _flag("--steps", ""):
        n = int(_flag("--steps", ""))
        cells = [dict(c, steps=n, measure_from=max(1, n // 3)) for c in cells]
    if "--dry-run" in sys.argv:
        import json

        print(json.dumps({"experiment": "distributed_sharding", "n_cells": len(cells), "cells": cells}, indent=1))
        return 0
    if smoke and "RANK" not in os.environ:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29518", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if cuda else "gloo")
    out = Path(_flag("--output", "") or common.RESULTS / "x8_fsdp2.jsonl")
    if smoke:
        cells = cells[:2]
    by_model: dict = {}
    for cell in cells:
        by_model.setdefault(cell.get("model_id", "model"), []).append(cell)
    for model_id, group in by_model.items():
        run_cohort(model_id, group, out, smoke=smoke)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
