"""Sharded data parallel (FSDP2 ``fully_shard`` per block, then the root) with STAC-R applied before sharding.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m experiments.benchmarks.distributed_sharding
    python -m experiments.benchmarks.distributed_sharding --smoke      # one rank, tiny model

Parity: experiments/benchmarks/distributed_sharding.py:1-362 of the reference project (bf16 parameters, torch AdamW,
per-rank peak via all_reduce MAX, cohorts up to 14B parameters).  Compression state stays per rank; the sharded
parameters are all-gathered by FSDP2 before the compressed layer's kernels see them.
"""

from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

import stacr_b200 as S
from stacr_b200.composition import transformer_blocks

from . import common
from .registry import EXPERIMENTS


def one_run(cell: dict, seed: int, smoke: bool = False) -> dict:
    from torch.distributed.fsdp import fully_shard

    cell = dict(cell)
    method = cell.pop("method")
    model_id, bs, seq = ("llama-tiny", 2, 64) if smoke else (cell["model_id"], cell["bs"], cell["seq"])
    steps, measure_from = (4, 1) if smoke else (30, 10)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    common.free_all()
    common.set_seed(seed)
    model = common.load_model(model_id, device, dtype=torch.bfloat16 if device == "cuda" else torch.float32)
    layers = common.stacr_on_blocks(model, dict(cell["stacr_cfg"], min_features=64 if smoke else 256)) if cell.get("stacr_cfg") else []
    for block in transformer_blocks(model):
        fully_shard(block)
    fully_shard(model)
    opt = torch.optim.AdamW(model.parameters(), lr=5e-5)
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
            "n_wrapped_layers": len(layers), "time_s": dt, "peak_GiB_max_rank": common.gib(float(peak)),
            "tokens_per_s_per_rank": bs * seq * measured / dt if dt > 0 and measured else None, "final_train_loss": float(loss), "status": "ok"}


def main() -> int:
    smoke = "--smoke" in sys.argv
    if smoke and "RANK" not in os.environ:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29518", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if cuda else "gloo")
    out = common.RESULTS / "x8_fsdp2.jsonl"
    cells = EXPERIMENTS["distributed_sharding"]["cells"]
    if smoke:
        cells = cells[:2]
    for cell in cells:
        try:
            rec = one_run(cell, 42, smoke=smoke)
        except torch.cuda.OutOfMemoryError:
            rec = {"method": cell["method"], "model": cell["model_id"], "status": "OOM"}
            torch.cuda.empty_cache()
        if dist.get_rank() == 0:
            if smoke:
                print(f"  smoke {rec['method']:14s} {rec.get('status')} loss={rec.get('final_train_loss')}", flush=True)
            else:
                common.emit(rec, out)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
