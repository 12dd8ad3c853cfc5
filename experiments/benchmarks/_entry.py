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


def arms(name: str) -> List[str]:
    """The distinct method names of the grid, in run order."""
    seen: List[str] = []
    for cell in cells(name):
        m = str(cell.get("method", cell.get("comparator", "")))
        if m not in seen:
            seen.append(m)
    return seen


def one(name: str, method: str, seed: int = 42, **overrides) -> dict:
    """Run the first cell of the grid whose method is ``method`` (keyword overrides replace cell fields) and return its row."""
    from . import grids

    for cell in cells(name):
        if str(cell.get("method")) == method:
            return grids._run_cell({**cell, **overrides}, seed)
    raise KeyError(f"grid {name!r} has no method {method!r}; choose from {arms(name)}")


def run_cohort(name: str, selector: str, seeds: Iterable[int] = (42,), output=None) -> List[dict]:
    """Run the cells whose method name contains ``selector`` (the ``--cohort`` flag of the command line)."""
    from . import common, grids
    from .registry import EXPERIMENTS

    rows = []
    for cell in EXPERIMENTS[name]["cells"]:
        if selector in str(cell.get("method", cell.get("comparator", ""))):
            for seed in seeds:
                row = grids._run_cell(dict(cell), seed)
                row["experiment"] = name
                rows.append(row)
                if output is not None and common._RECORDER is None:
                    common.emit(row, output)
    if not rows:
        raise KeyError(f"selector {selector!r} matches no cell of {name!r}")
    return rows


def main(name: str, argv: Optional[List[str]] = None) -> int:
    from .__main__ import main as cli

    return cli(["run", name, *(argv if argv is not None else __import__("sys").argv[1:])])


def bind(namespace: dict, name: str) -> None:
    """Give a grid module its standard entry points: ``NAME``, ``cells``, ``rows``, ``arms``, ``run``, ``run_cohort``,
    ``one`` and ``main``, all bound to grid ``name`` (names the module has already defined are left alone)."""

    def _cells():
        return cells(name)

    def _arms():
        return arms(name)

    def _run(seeds=(42,), output=None):
        return run(name, seeds, output)

    def _run_cohort(selector, seeds=(42,), output=None):
        return run_cohort(name, selector, seeds, output)

    def _one(method, seed=42, **overrides):
        return one(name, method, seed, **overrides)

    def _main(argv=None) -> int:
        return main(name, argv)

    bound = {"NAME": name, "cells": _cells, "rows": _cells, "arms": _arms, "run": _run, "run_cohort": _run_cohort, "one": _one, "main": _main}
    for key, value in bound.items():
        namespace.setdefault(key, value)
