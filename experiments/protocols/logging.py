"""Run directory writer: ``config.json``, ``metrics.jsonl``, ``profile.jsonl``, ``final.json``.

Rank 0 logs; other ranks get ``NullLogger`` (parity: experiments/protocols/logging.py:29-73 of the reference project).
"""

from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Any, Dict


class RunLogger:
    def __init__(self, output_dir: str | Path):
        self.dir = Path(output_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self._t0 = time.time()

    @property
    def profile_path(self) -> str:
        return str(self.dir / "profile.jsonl")

    def write_config(self, config: Dict[str, Any]) -> None:
        (self.dir / "config.json").write_text(json.dumps(config, indent=2, default=str), encoding="utf-8")

    def log(self, record: Dict[str, Any]) -> None:
        with (self.dir / "metrics.jsonl").open("a", encoding="utf-8") as fh:
            fh.write(json.dumps({"t": time.time() - self._t0, **record}, default=str) + "\n")

    def write_final(self, record: Dict[str, Any]) -> None:
        (self.dir / "final.json").write_text(json.dumps(record, indent=2, default=str), encoding="utf-8")


class NullLogger:
    profile_path = None

    def write_config(self, config):
        pass

    def log(self, record):
        pass

    def write_final(self, record):
        pass
