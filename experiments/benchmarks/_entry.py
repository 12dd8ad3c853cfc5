"""Shared body of the per-grid entry modules (``python -m experiments.benchmarks.<grid>``).

Every grid is declared once, as data, in ``registry.EXPERIMENTS`` and executed by ``grids.run_experiment``.  The
entry modules give each grid the module path scripts and papers cite, and a ``main`` that accepts the same flags
as ``python -m experiments.benchmarks run <grid>``.
"""

from __future__ import annotations

from typing import Iterable, List, Optional


def cells(name: str) -> List[dict]:
    """The grid's cells (method, model, batch shape, compression options) as declared in the registry."""
    from .registry import EXPERIMENTS

    return [dict(c) for c in EXPERIMENTS[name]["cells"]]


def describe(name: str) -> dict:
    from .registry import EXPERIMENTS

    meta = EXPERIMENTS[name]
    return {k: v for k, v in meta.items() if k != "cells"} | {"n_cells": len(meta["cells"])}


def run(name: str, seeds: Iterable[int] = (42,), output=None) -> List[dict]:
    """Run the grid in this process and return its rows (also appended to the grid's result file)."""
    from . import grids

    return grids.run_experiment(name, seeds, output)


def main(name: str, argv: Optional[List[str]] = None) -> int:
    from .__main__ import main as cli

    return cli(["run", name, *(argv if argv is not None else __import__("sys").argv[1:])])
