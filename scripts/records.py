"""Turn benchmark JSON lines into measurement records and cohort rows.

    python -m scripts.records add bench_line.json [more.json ...] [--platform b200] [--cohort headline_b200]

Each input file holds the single JSON line printed by the repo's benchmark.  The record id is the SHA-256 of the
canonical row, so adding a file twice changes nothing.  ``results/records.jsonl`` is kept sorted by id and
``results/cohorts.csv`` gets one row per record (method = the ``impl`` field).
"""

from __future__ import annotations

import argparse
import csv
import hashlib
import json
from pathlib import Path

from .evidence import REPO, canonical, read_jsonl

COHORT_FIELDS = ("cohort", "method", "seed", "accuracy", "ppl", "peak_gib", "time_s", "tokens_per_s", "cosine", "timing_excluded")
METHOD_NAMES = {"reference": "baseline"}


def bench_row(line: dict, cohort: str) -> dict:
    cfg = line.get("config", {})
    mem = line.get("memory", {})
    row = {
        "tag": "b200_" + str(cfg.get("model", "model")).split(" ")[0], "cohort": cohort, "method": METHOD_NAMES.get(line.get("impl"), line.get("impl", "stacr_b200")),
        "model": cfg.get("model"), "bs": cfg.get("global_batch"), "seq": cfg.get("seq_len"), "steps": line.get("steps"), "steps_measured": line.get("steps"),
        "world_size": line.get("n_gpus", 1), "dtype": line.get("dtype"), "dataset": "synthetic", "optimizer_actual": cfg.get("optimizer"),
        "stacr_cfg": cfg.get("stacr"), "seed": 0, "tokens_per_s": line.get("value"), "time_s": line.get("ms_per_step", 0.0) * line.get("steps", 0) / 1e3,
        "ms_per_step": line.get("ms_per_step"), "e2e_tokens_per_s": (line.get("e2e") or {}).get("value"), "gpu_launches": line.get("gpu_launches"),
        "clocks": line.get("clocks"),
    }
    if mem.get("peak_allocated_gb") is not None:
        row["peak_GiB"] = mem["peak_allocated_gb"] * 1e9 / 2 ** 30
        row["peak_bytes"] = int(mem["peak_allocated_gb"] * 1e9)
    if mem.get("saved_activation_gb_wrapped_layers") is not None:
        row["stored_MiB"] = mem["saved_activation_gb_wrapped_layers"] * 1e9 / 2 ** 20
    return {k: v for k, v in row.items() if v is not None}


def add(paths, data: Path, platform: str, cohort: str, experiment: str) -> int:
    results = Path(data) / "results"
    results.mkdir(parents=True, exist_ok=True)
    store = results / "records.jsonl"
    records = {r["record_id"]: r for r in read_jsonl(store)} if store.is_file() else {}
    before = len(records)
    for path in paths:
        text = Path(path).read_text(encoding="utf-8").strip().splitlines()
        line = json.loads(next(t for t in reversed(text) if t.startswith("{")))
        if "value" not in line:
            continue
        row = bench_row(line, cohort)
        rid = hashlib.sha256(canonical(row).encode()).hexdigest()
        records[rid] = {"record_id": rid, "platform": platform, "experiments": [experiment], "flags": [], "row": row}
    with store.open("w", encoding="utf-8") as fh:
        for rid in sorted(records):
            fh.write(canonical(records[rid]) + "\n")
    with (results / "cohorts.csv").open("w", encoding="utf-8", newline="") as fh:
        writer = csv.DictWriter(fh, fieldnames=COHORT_FIELDS)
        writer.writeheader()
        for rid in sorted(records):
            row = records[rid]["row"]
            writer.writerow({"cohort": row.get("cohort", cohort), "method": row["method"], "seed": row.get("seed", 0), "accuracy": "", "ppl": "",
                             "peak_gib": row.get("peak_GiB", ""), "time_s": row.get("time_s", ""), "tokens_per_s": row.get("tokens_per_s", ""),
                             "cosine": "", "timing_excluded": "false"})
    return len(records) - before


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    sub = parser.add_subparsers(dest="command", required=True)
    p = sub.add_parser("add")
    p.add_argument("files", nargs="+")
    p.add_argument("--data", type=Path, default=REPO / "paper_data")
    p.add_argument("--platform", default="b200")
    p.add_argument("--cohort", default="headline_b200")
    p.add_argument("--experiment", default="headline")
    args = parser.parse_args(argv)
    print(f"added {add(args.files, args.data, args.platform, args.cohort, args.experiment)} record(s)")


if __name__ == "__main__":
    main()
