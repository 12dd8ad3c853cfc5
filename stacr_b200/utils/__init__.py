"""Small host-side helpers: CLI override parsing, seeding, YAML/CSV IO, device resolution.

Behavioural parity: stacr/utils.py:14-74 of the reference project (only ``true``/``false`` become
booleans in ``--set`` overrides; ``on``/``off``/``yes``/``no`` stay strings).
"""

from __future__ import annotations

import csv
import random
import re
from pathlib import Path
from typing import Iterable

import numpy as np
import torch
import yaml


def _make_override_loader():
    class Loader(yaml.SafeLoader):
        pass

    # private copy of the implicit resolvers without YAML 1.1's on/off/yes/no booleans
    Loader.yaml_implicit_resolvers = {
        first: [(tag, rx) for tag, rx in rules if tag != "tag:yaml.org,2002:bool"]
        for first, rules in yaml.SafeLoader.yaml_implicit_resolvers.items()
    }
    Loader.add_implicit_resolver("tag:yaml.org,2002:bool", re.compile(r"^(?:true|false)$", re.IGNORECASE), list("tTfF"))
    return Loader


_OverrideLoader = _make_override_loader()


def parse_override(value: str):
    """Parse one ``KEY=VALUE`` value with YAML typing, except that only true/false are booleans."""
    return yaml.load(value, Loader=_OverrideLoader)


def set_seed(seed: int) -> None:
    seed = int(seed)
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def load_yaml(path: str | Path) -> dict:
    with open(path, "r", encoding="utf-8") as fh:
        data = yaml.safe_load(fh)
    if not isinstance(data, dict):
        raise ValueError(f"Configuration {path} must be a YAML mapping")
    return data


def write_csv(path: str | Path, rows: Iterable[dict]) -> None:
    rows = list(rows)
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    if not rows:
        path.write_text("", encoding="utf-8")
        return
    columns: dict[str, None] = {}
    for row in rows:
        columns.update(dict.fromkeys(row))
    with path.open("w", newline="", encoding="utf-8") as fh:
        writer = csv.DictWriter(fh, fieldnames=list(columns))
        writer.writeheader()
        writer.writerows(rows)


def device_from_config(value: str = "auto") -> torch.device:
    if value == "auto":
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")
    device = torch.device(value)
    if device.type == "cuda" and not torch.cuda.is_available():
        raise RuntimeError("CUDA was requested but no CUDA device is available")
    return device
