"""``python -m stacr reproduce list | run <profile> [--seeds --steps --device --output --dry-run --set K=V] | openwebtext | bounds``.

Profiles live in ``configs/protocols.json``.  A profile names its ``world_size``; when it is greater than one the
command must be launched with ``torchrun`` and the matching number of ranks.
Parity: experiments/protocols/__main__.py:1-199 of the reference project.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path


def profiles() -> dict:
    from importlib.resources import files

    return json.loads(files("configs").joinpath("protocols.json").read_text(encoding="utf-8"))["profiles"]


def make_config(raw: dict, seed: int, overrides: dict):
    from stacr_b200.utils import parse_override

    from .training import ConvergenceConfig

    data = dict(raw["config"])
    data["seed"] = seed
    for key, value in overrides.items():
        data[key] = parse_override(value) if isinstance(value, str) else value
    cfg = ConvergenceConfig.from_raw(data)
    if cfg.use_ddp and cfg.use_tensor_parallel:
        raise ValueError("Select DDP or tensor parallelism")
    return cfg


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)
    listing = sub.add_parser("list")
    listing.add_argument("--group")
    run = sub.add_parser("run")
    run.add_argument("profile")
    run.add_argument("--seeds", type=int, nargs="+")
    run.add_argument("--steps", type=int)
    run.add_argument("--device")
    run.add_argument("--output", type=Path, default=Path("outputs/protocols"))
    run.add_argument("--dry-run", action="store_true")
    run.add_argument("--set", action="append", default=[], metavar="KEY=VALUE")
    sub.add_parser("openwebtext", help="paired baseline/STAC-R transfer smoke protocol")
    sub.add_parser("bounds", help="per-layer gradient-bound probe on a saved checkpoint")
    args, rest = parser.parse_known_args(argv)
    table = profiles()
    if args.command == "list":
        for name, prof in table.items():
            if args.group and prof["group"] != args.group:
                continue
            print(f"{name:44s} [{prof['group']}] world={prof.get('world_size', 1)} {prof.get('description', '')}")
        return 0
    if args.command == "openwebtext":
        from .openwebtext_transfer import main as owt_main

        return owt_main(rest)
    if args.command == "bounds":
        from scripts.theorem_probe import main as probe_main

        return probe_main(rest)
    if args.profile not in table:
        parser.error(f"unknown profile {args.profile!r}; see `reproduce list`")
    prof = table[args.profile]
    overrides = {}
    for item in args.set:
        key, sep, value = item.partition("=")
        if not sep:
            parser.error("--set needs KEY=VALUE")
        overrides[key] = value
    if args.steps is not None:
        overrides["max_steps"] = args.steps
    if args.device:
        overrides["device"] = args.device
    seeds = args.seeds or prof.get("seeds", [42])
    if args.dry_run:
        print(json.dumps({"profile": args.profile, "group": prof["group"], "world_size": prof.get("world_size", 1), "seeds": seeds,
                          "configs": [make_config(prof, s, overrides).to_dict() for s in seeds]}, indent=2, default=str))
        return 0
    for key, value in prof.get("environment", {}).items():
        os.environ.setdefault(key, str(value))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    need = int(prof.get("world_size", 1))
    if world != need:
        print(f"profile {args.profile} needs world_size={need} but WORLD_SIZE={world}; launch with "
              f"`python -m torch.distributed.run --nproc-per-node {need} -m stacr reproduce run {args.profile}`", file=sys.stderr)
        return 2
    import torch
    import torch.distributed as dist

    from .logging import NullLogger, RunLogger
    from .training import run_convergence_experiment

    if need > 1:
        from stacr_b200.parallel import init_distributed

        init_distributed()
    rank = dist.get_rank() if dist.is_initialized() else 0
    code = 0
    for seed in seeds:
        cfg = make_config(prof, seed, overrides)
        if cfg.task == "ogbn-arxiv":
            # node classification runs in the graph protocol (full-batch GCN; synthetic graph when the dataset is absent)
            from .graph import run as run_graph

            epochs = cfg.epochs if cfg.max_steps >= (1 << 62) else min(cfg.epochs, cfg.max_steps)
            final = run_graph(method="stacr" if cfg.method == "stacr" else "baseline", epochs=epochs, seed=seed, rank=cfg.rank, budget=cfg.stacr_residual_budget)
            if rank == 0:
                RunLogger(args.output / args.profile / f"seed{seed}").write_final(final)
                print(json.dumps({"run_tag": cfg.run_tag, **{k: final[k] for k in list(final)[:6]}}, default=str))
            continue
        logger = RunLogger(args.output / args.profile / f"seed{seed}") if rank == 0 else NullLogger()
        try:
            final = run_convergence_experiment(cfg, logger)
            if rank == 0:
                print(json.dumps({k: final[k] for k in ("run_tag", "status", "steps", "train_loss_last", "tokens_per_second", "peak_allocated_bytes") if k in final}))
            if not str(final.get("status", "ok")).startswith("ok"):
                code = 1
        except Exception as exc:  # noqa: BLE001
            logger.write_final({"status": "error", "error": f"{type(exc).__name__}: {exc}"})
            raise
    if dist.is_initialized():
        dist.destroy_process_group()
    return code


if __name__ == "__main__":
    raise SystemExit(main())
