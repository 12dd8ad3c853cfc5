"""Command line: ``python -m stacr {doctor,train,fidelity,reproduce,benchmarks}``.

Each sub-command is one handler in ``_HANDLERS``.  ``reproduce`` and ``benchmarks`` own their argument parsing (the experiment
packages), so they are dispatched on the first word before this module's parser exists; ``train`` and ``fidelity`` share one
pipeline: YAML (path or packaged preset) -> ``--set`` overrides -> explicit flags -> ``--demo`` caps -> validation -> run ->
CSV + resolved settings as JSON.  Model libraries are imported only by the handlers that need them.

Surface parity: stacr/cli.py:13-137 of the reference project (same sub-commands, flags, override typing and output files);
``doctor`` additionally reports the sm_100a kernel library, the compute capability of each GPU and the collective back ends.
"""

from __future__ import annotations

import argparse
import json
import platform
import sys
from importlib import metadata
from pathlib import Path

_REPORTED_PACKAGES = ("stacr", "stacr-b200", "torch", "transformers", "datasets", "accelerate", "bitsandbytes", "peft", "galore-torch")
_DEMO_CAPS = {"steps": 5, "max_examples": 64, "max_eval_examples": 16}
_RUN_COMMANDS = {"train": "Train a configuration", "fidelity": "Compare paired gradients"}


# ------------------------------------------------------------------------------------------------ doctor
def _installed_version(package: str):
    try:
        return metadata.version(package)
    except metadata.PackageNotFoundError:
        return None


def _kernel_library_report() -> dict:
    from .ops import _lib, build

    path = _lib.lib_path()
    report = {"path": str(path) if path.exists() else None, "sources_newer_than_library": None}
    if path.exists():
        try:
            report["sources_newer_than_library"] = bool(build.is_stale())
        except OSError:
            pass
    return report


def doctor() -> dict:
    import torch
    import torch.distributed as dist

    gpus = []
    for index in range(torch.cuda.device_count()):
        props = torch.cuda.get_device_properties(index)
        gpus.append({"name": props.name, "memory_gib": props.total_memory / 1024**3, "capability": [props.major, props.minor],
                     "multiprocessors": props.multi_processor_count})
    library = _kernel_library_report()
    return {
        "python": platform.python_version(),
        "platform": platform.system(),
        "libraries": {name: _installed_version(name) for name in _REPORTED_PACKAGES},
        "cuda_available": torch.cuda.is_available(),
        "cuda_runtime": torch.version.cuda,
        "kernel_library": library["path"],
        "kernel_library_stale": library["sources_newer_than_library"],
        "collectives": {"nccl": dist.is_available() and dist.is_nccl_available(), "gloo": dist.is_available() and dist.is_gloo_available()},
        "gpus": gpus,
    }


# ------------------------------------------------------------------------------------------------ settings
def resolve_config(name):
    """A YAML path, or the name of a packaged preset under ``configs/`` (with or without ``.yaml``)."""
    from importlib.resources import files

    as_path = Path(name)
    if as_path.is_file():
        return as_path
    stem = name if str(name).endswith(".yaml") else f"{name}.yaml"
    packaged = files("configs").joinpath(stem)
    if not packaged.is_file():
        raise ValueError(f"Config {name!r} not found; pass a YAML path or a packaged preset name")
    return packaged


def _apply_overrides(settings: dict, pairs: list[str], fail) -> None:
    from .utils import parse_override

    for pair in pairs:
        key, equals, raw = pair.partition("=")
        if not (key and equals):
            fail("--set needs KEY=VALUE")
        settings[key] = parse_override(raw)


def _settings_from(ns: argparse.Namespace, fail) -> dict:
    """The validated settings of a ``train`` / ``fidelity`` invocation; later sources win (file < --set < flags < --demo caps)."""
    from .training import validate_config
    from .utils import load_yaml

    settings = load_yaml(resolve_config(ns.config))
    _apply_overrides(settings, ns.set, fail)
    settings.update({key: value for key in ("steps", "seed", "device") if (value := getattr(ns, key)) is not None})
    if ns.demo:
        settings.update({key: min(int(settings.get(key, cap)), cap) for key, cap in _DEMO_CAPS.items()})
    return validate_config(settings)


# ------------------------------------------------------------------------------------------------ handlers
def _cmd_doctor(ns, fail) -> None:
    print(json.dumps(doctor(), indent=2))


def _cmd_run(ns, fail) -> None:
    from .training import gradient_fidelity, run_config
    from .utils import write_csv

    settings = _settings_from(ns, fail)
    if ns.dry_run:
        print(json.dumps(settings, indent=2))
        return
    target = Path(ns.output) if ns.output else Path("outputs") / f"{Path(ns.config).stem}_{ns.command}_seed{settings['seed']}.csv"
    target.parent.mkdir(parents=True, exist_ok=True)
    target.with_suffix(".config.json").write_text(json.dumps(settings, indent=2), encoding="utf-8")
    row = (gradient_fidelity if ns.command == "fidelity" else run_config)(settings)
    write_csv(target, [row])
    print(json.dumps(row, indent=2, default=str))


def _delegate(module: str):
    def run(rest: list[str]):
        from importlib import import_module

        return import_module(module).main(rest)
    return run


_DELEGATED = {"reproduce": _delegate("experiments.protocols.__main__"), "benchmarks": _delegate("experiments.benchmarks.__main__")}
_HANDLERS = {"doctor": _cmd_doctor, **{name: _cmd_run for name in _RUN_COMMANDS}}


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="STAC-R training, integration checks and experiments.")
    commands = parser.add_subparsers(dest="command", required=True)
    commands.add_parser("doctor", help="Report library versions and available GPUs")
    commands.add_parser("benchmarks", help="List or run measurement grids")
    commands.add_parser("reproduce", help="List or run training protocols")
    for name, summary in _RUN_COMMANDS.items():
        p = commands.add_parser(name, help=summary)
        p.add_argument("--config", required=True)
        for flag, kind in (("--steps", int), ("--seed", int), ("--device", str)):
            p.add_argument(flag, type=kind)
        p.add_argument("--demo", action="store_true")
        p.add_argument("--dry-run", action="store_true", help="Print resolved settings without loading data/models")
        p.add_argument("--output", help="CSV output; resolved settings are saved alongside it as JSON")
        p.add_argument("--set", action="append", default=[], metavar="KEY=VALUE", help="Override a YAML setting")
    return parser


def main(argv=None):
    words = list(sys.argv[1:] if argv is None else argv)
    if words and words[0] in _DELEGATED:
        return _DELEGATED[words[0]](words[1:])
    parser = _parser()
    ns = parser.parse_args(words)
    _HANDLERS[ns.command](ns, parser.error)
    return None


if __name__ == "__main__":
    raise SystemExit(main())
