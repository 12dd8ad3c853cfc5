"""Launcher for an INSTANT run.

Parity: comparators/instant_wrapper.py (``run_instant(command, cwd)``).  ``run_instant`` executes an external
INSTANT command line and returns its exit code; ``run_instant_language`` / ``run_instant_classification`` call the
in-tree comparator of ``stacr_b200.comparators.instant`` in this process instead.
"""

from __future__ import annotations

import subprocess
from pathlib import Path


def run_instant(command: list[str], cwd: str | Path | None = None) -> int:
    if not command:
        raise ValueError("run_instant needs a command line")
    return subprocess.call([str(c) for c in command], cwd=str(cwd) if cwd is not None else None)


def run_instant_language(argv: list[str] | None = None) -> dict:
    from .instant import train_language

    return train_language.main(argv)


def run_instant_classification(argv: list[str] | None = None) -> dict:
    from .instant import train_classification

    return train_classification.main(argv)
