"""Generic runner for the declaratively registered grids: turn a cell dict into a ``common`` call and emit its row."""

from __future__ import annotations

import os
from typing import Iterable

import torch

from . import common
from .registry import EXPERIMENTS

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _complement(k):
    return (lambda i, _k=k: i % _k != 0) if k else None


def _run_cell(cell: dict, seed: int) -> dict:
    cell = dict(cell)
    kind = cell.pop("kind", "train")
    overrides = common.PARAMETERS
    for key in ("steps", "model_id", "bs", "seq", "eval_batches", "measure_from", "dataset", "attn_impl"):
        if key in overrides:
            cell[key] = overrides[key]
    if isinstance(cell.get("model_dtype"), str):
        cell["model_dtype"] = _DTYPES[cell["model_dtype"]]
    comparator = cell.pop("comparator", None)
    if kind == "fidelity":
        cfg = dict(cell.pop("stacr_cfg"))
        for k in ("single_model",):
            cell.pop(k, None)
        row = common.gradient_fidelity(cell.pop("model_id"), cfg, seed=seed, **{k: v for k, v in cell.items() if k in ("bs", "seq", "steps")})
        if comparator:
            row["comparator"] = comparator
        return row
    k = cell.pop("complement", None)
    if k:
        cell["stacr_block_pred"] = _complement(k)
    if comparator and comparator not in ("stacr", "turbo"):
        cell["basis_comparator"] = comparator
    if cell.get("steps") and cell.get("measure_from", 20) >= cell["steps"]:
        cell["measure_from"] = max(0, cell["steps"] // 3)
    return common.run_config(cell.pop("method"), seed, **cell)


def run_experiment(name: str, seeds: Iterable[int] = (42,), output: str | os.PathLike | None = None) -> list[dict]:
    meta = EXPERIMENTS[name]
    out = output or (common.RESULTS / f"{name}.jsonl")
    rows = []
    stopped: set = set()            # (method, model) pairs of an ascending probe that already ran out of memory
    for cell in meta["cells"]:
        for seed in (seeds if meta.get("seeds") else list(seeds)[:1]):
            probe_key = (cell.get("method"), cell.get("model_id"), seed) if cell.get("probe") == "ascending" else None
            if probe_key in stopped:
                rows.append({"method": cell.get("method"), "model": cell.get("model_id"), "bs": cell.get("bs"), "seed": seed, "fits": False,
                             "status": "skipped_larger_than_first_failure", "experiment": name})
                continue
            try:
                row = _run_cell(cell, seed)
            except torch.cuda.OutOfMemoryError:
                row = {"method": cell.get("method"), "model": cell.get("model_id"), "seed": seed, "status": "OOM"}
                torch.cuda.empty_cache()
            except FloatingPointError as exc:
                row = {"method": cell.get("method"), "model": cell.get("model_id"), "seed": seed, "status": "nonfinite", "error": str(exc)}
            row["experiment"] = name
            if probe_key is not None:
                row["fits"] = row.get("status") == "ok"
                if not row["fits"]:
                    stopped.add(probe_key)
            rows.append(row)
            if common._RECORDER is None:
                common.emit(row, out)
    return rows
