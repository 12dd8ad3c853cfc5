"""Command line: ``python -m stacr {doctor,train,fidelity,reproduce,benchmarks}``.

Parity: stacr/cli.py:13-137 of the reference project.  ``reproduce`` and ``benchmarks`` are
delegated to the experiment packages before argument parsing; model libraries are imported only by
the commands that need them.
"""

from __future__ import annotations

import argparse
import importlib.metadata
import json
import platform
import sys
from pathlib import Path


def doctor() -> dict:
    import torch

    from .ops import _lib

    libs = {}
    for name in ("stacr", "stacr-b200", "torch", "transformers", "datasets", "accelerate", "bitsandbytes", "peft", "galore-torch"):
        try:
            libs[name] = importlib.metadata.version(name)
        except importlib.metadata.PackageNotFoundError:
            libs[name] = None
    return {
        "python": platform.python_version(),
        "platform": platform.system(),
        "libraries": libs,
        "cuda_available": torch.cuda.is_available(),
        "cuda_runtime": torch.version.cuda,
        "kernel_library": str(_lib.lib_path()) if _lib.lib_path().exists() else None,
        "gpus": [
            {"name": torch.cuda.get_device_name(i), "memory_gib": torch.cuda.get_device_properties(i).total_memory / 1024**3,
             "capability": list(torch.cuda.get_device_capability(i))}
            for i in range(torch.cuda.device_count())
        ],
    }


def resolve_config(name):
    """A YAML path, or the name of a packaged preset under ``configs/``."""
    from importlib.resources import files

    path = Path(name)
    if path.is_file():
        return path
    preset = files("configs").joinpath(name if name.endswith(".yaml") else f"{name}.yaml")
    if preset.is_file():
        return preset
    raise ValueError(f"Config {name!r} not found; pass a YAML path or a packaged preset name")


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="STAC-R training, integration checks and experiments.")
    sub = parser.add_subparsers(dest="command", required=True)
    sub.add_parser("doctor", help="Report library versions and available GPUs")
    sub.add_parser("benchmarks", help="List or run measurement grids")
    sub.add_parser("reproduce", help="List or run training protocols")
    for name, text in (("train", "Train a configuration"), ("fidelity", "Compare paired gradients")):
        run = sub.add_parser(name, help=text)
        run.add_argument("--config", required=True)
        run.add_argument("--steps", type=int)
        run.add_argument("--seed", type=int)
        run.add_argument("--device")
        run.add_argument("--demo", action="store_true")
        run.add_argument("--dry-run", action="store_true", help="Print resolved settings without loading data/models")
        run.add_argument("--output", help="CSV output; resolved settings are saved alongside it as JSON")
        run.add_argument("--set", action="append", default=[], metavar="KEY=VALUE", help="Override a YAML setting")
    return parser


def main(argv=None):
    args = list(sys.argv[1:] if argv is None else argv)
    if args[:1] == ["reproduce"]:
        from experiments.protocols.__main__ import main as protocol_main

        return protocol_main(args[1:])
    if args[:1] == ["benchmarks"]:
        from experiments.benchmarks.__main__ import main as benchmark_main

        return benchmark_main(args[1:])
    parser = _parser()
    ns = parser.parse_args(args)
    if ns.command == "doctor":
        print(json.dumps(doctor(), indent=2))
        return None
    from .training import gradient_fidelity, run_config, validate_config
    from .utils import load_yaml, parse_override, write_csv

    config = load_yaml(resolve_config(ns.config))
    for item in ns.set:
        key, sep, value = item.partition("=")
        if not sep or not key:
            parser.error("--set needs KEY=VALUE")
        config[key] = parse_override(value)
    for key in ("steps", "seed", "device"):
        if getattr(ns, key) is not None:
            config[key] = getattr(ns, key)
    if ns.demo:
        for key, cap, default in (("steps", 5, 5), ("max_examples", 64, 64), ("max_eval_examples", 16, 16)):
            config[key] = min(int(config.get(key, default)), cap)
    config = validate_config(config)
    if ns.dry_run:
        print(json.dumps(config, indent=2))
        return None
    output = Path(ns.output or f"outputs/{Path(ns.config).stem}_{ns.command}_seed{config['seed']}.csv")
    output.parent.mkdir(parents=True, exist_ok=True)
    output.with_suffix(".config.json").write_text(json.dumps(config, indent=2), encoding="utf-8")
    result = gradient_fidelity(config) if ns.command == "fidelity" else run_config(config)
    write_csv(output, [result])
    print(json.dumps(result, indent=2, default=str))
    return None


if __name__ == "__main__":
    raise SystemExit(main())
