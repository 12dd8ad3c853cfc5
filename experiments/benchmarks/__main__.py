"""``python -m experiments.benchmarks list|run <experiment> [--dry-run --plan-output FILE --steps N ...]``.

``--dry-run`` replaces every measurement cell with a recorder and prints (or writes) the full cell plan without
touching a model, a dataset or a GPU.  Parity: experiments/benchmarks/__main__.py:1-365 of the reference project.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from .registry import EXPERIMENTS


def _jsonable(value):
    if isinstance(value, dict):
        return {k: _jsonable(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_jsonable(v) for v in value]
    if callable(value):
        return getattr(value, "__name__", "callable")
    if isinstance(value, (int, float, str, bool)) or value is None:
        return value
    return str(value)


def _plan(name: str, seeds) -> list[dict]:
    from . import common, grids

    plan: list[dict] = []

    def record(**cell):
        plan.append(_jsonable(cell))
        return {"status": "planned", **{k: v for k, v in cell.items() if isinstance(v, (int, float, str, bool, type(None)))}}

    common.set_recorder(record)
    try:
        if EXPERIMENTS[name]["module"] == "grids":
            grids.run_experiment(name, seeds)
        else:
            for cell in EXPERIMENTS[name]["cells"]:
                for seed in seeds:
                    record(seed=seed, launcher="torchrun", **cell)
    finally:
        common.set_recorder(None)
    return plan


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)
    listing = sub.add_parser("list", help="List available experiments")
    listing.add_argument("--json", action="store_true")
    run = sub.add_parser("run", help="Run one experiment; --dry-run prints its full cell plan")
    run.add_argument("experiment", choices=sorted(EXPERIMENTS))
    run.add_argument("--dry-run", action="store_true")
    run.add_argument("--plan-output", type=Path)
    run.add_argument("--output", type=Path)
    run.add_argument("--append", action="store_true", help="Append a distinct run ID to an existing output file")
    run.add_argument("--steps", type=int)
    run.add_argument("--seeds", type=int, nargs="+")
    run.add_argument("--model", dest="model_id")
    run.add_argument("--batch-size", dest="bs", type=int)
    run.add_argument("--seq-length", dest="seq", type=int)
    run.add_argument("--eval-batches", type=int)
    run.add_argument("--measure-from", type=int)
    run.add_argument("--device", choices=("cuda", "cpu"))
    run.add_argument("--optimizer", choices=("adamw8bit", "adamw"))
    run.add_argument("--dataset", choices=("synthetic", "wikitext", "openwebtext"))
    run.add_argument("--attention", dest="attn_impl", choices=("eager", "sdpa", "flash_attention_2"))
    run.add_argument("--cohort", action="append", default=[], help="Experiment-specific selector; a substring of the cell's method name")
    args = parser.parse_args(argv)
    if args.command == "list":
        if args.json:
            print(json.dumps({k: {x: y for x, y in v.items() if x != "cells"} | {"n_cells": len(v["cells"])} for k, v in EXPERIMENTS.items()}, indent=2))
        else:
            for name, meta in sorted(EXPERIMENTS.items()):
                print(f"{name:27s} {meta['description']}")
        return 0
    from . import common, grids

    name = args.experiment
    common.configure(steps=args.steps, model_id=args.model_id, bs=args.bs, seq=args.seq, eval_batches=args.eval_batches,
                     measure_from=args.measure_from, device=args.device, optimizer=args.optimizer, dataset=args.dataset, attn_impl=args.attn_impl)
    seeds = args.seeds or ([42, 123, 456] if EXPERIMENTS[name].get("seeds") else [42])
    if args.cohort:
        meta = EXPERIMENTS[name]
        meta["cells"] = [c for c in meta["cells"] if any(sel in str(c.get("method", c.get("comparator", ""))) for sel in args.cohort)]
        if not meta["cells"]:
            parser.error(f"--cohort {args.cohort} matches no cell of {name}")
    if args.dry_run:
        plan = _plan(name, seeds)
        if not plan:
            print(f"{name}: empty plan", file=sys.stderr)
            return 1
        text = json.dumps({"experiment": name, "cells": plan, "n_cells": len(plan)}, indent=2)
        if args.plan_output:
            args.plan_output.parent.mkdir(parents=True, exist_ok=True)
            args.plan_output.write_text(text, encoding="utf-8")
        else:
            print(text)
        return 0
    if EXPERIMENTS[name]["module"] != "grids":
        print(f"{name} is a multi-process grid: launch `python -m torch.distributed.run --nproc-per-node N -m experiments.benchmarks.{EXPERIMENTS[name]['module']}`")
        return 2
    if args.output and args.output.exists() and not args.append:
        parser.error(f"{args.output} exists; pass --append to add a new run to it")
    rows = grids.run_experiment(name, seeds, args.output)
    return 0 if all(r.get("status") in ("ok", "OOM", None) or "mean_cosine" in r for r in rows) else 1


if __name__ == "__main__":
    raise SystemExit(main())
