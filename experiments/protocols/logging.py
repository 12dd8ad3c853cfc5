"""Run directory writer: ``config.json``, ``metrics.jsonl``, ``profile.jsonl``, ``final.json``.

Rank 0 logs; other ranks get ``NullLogger`` (parity: experiments/protocols/logging.py:29-73 of the reference project).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
import time
from pathlib import Path
from typing import Any, Dict


@dataclass
class TrainConfig:
    """Defaults of the small vision-style demo loop that shares this logger (epochs, batch size, SGD settings, loader workers)."""

    epochs: int = 3
    batch_size: int = 128
    lr: float = 0.01
    momentum: float = 0.9
    num_workers: int = 2


class RunLogger:
    """One run directory: ``config.json``, ``metrics.jsonl`` (one line per step), ``profile.jsonl``, ``final.json``."""

    def __init__(self, output_dir: str | Path):
        self.dir = self.run_dir = Path(output_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self._t0 = time.time()
        self.config_path, self.metrics_path, self.final_path = self.dir / "config.json", self.dir / "metrics.jsonl", self.dir / "final.json"
        self.metrics_path.touch(exist_ok=True)
        (self.dir / "profile.jsonl").touch(exist_ok=True)

    @property
    def profile_path(self) -> str:
        return str(self.dir / "profile.jsonl")

    def log_metrics(self, payload: Dict[str, Any]) -> None:
        self.log(payload)

    def log_profile(self, payload: Dict[str, Any]) -> None:
        with open(self.profile_path, "a", encoding="utf-8") as fh:
            fh.write(json.dumps(payload, default=str) + "\n")

    def write_config(self, config: Dict[str, Any]) -> None:
        (self.dir / "config.json").write_text(json.dumps(config, indent=2, default=str), encoding="utf-8")

    def log(self, record: Dict[str, Any]) -> None:
        with (self.dir / "metrics.jsonl").open("a", encoding="utf-8") as fh:
            fh.write(json.dumps({"t": time.time() - self._t0, **record}, default=str) + "\n")

    def write_final(self, record: Dict[str, Any]) -> None:
        (self.dir / "final.json").write_text(json.dumps(record, indent=2, default=str), encoding="utf-8")


class NullLogger:
    profile_path = None
    run_dir = dir = None

    def __init__(self, run_dir=None):
        pass

    def log_metrics(self, payload):
        pass

    def log_profile(self, payload):
        pass

    def write_config(self, config):
        pass

    def log(self, record):
        pass

    def write_final(self, record):
        pass
