"""Summaries of measurement records and recomputation of cohort statistics.

A record is one JSON line ``{"record_id", "platform", "experiments": [...], "flags": [...], "row": {...}}``.
``summary`` groups records that share hardware, protocol and method settings and reports per-metric statistics
over independent seeds (several executions of one seed are averaged first, so they do not inflate n).
Records carrying a validity flag are left out of the statistics unless ``--include-flagged`` is given; quality
metrics (perplexity, accuracy) have a second, stricter flag list.

    python -m scripts.evidence list
    python -m scripts.evidence summary --experiment headline --platform b200
    python -m scripts.evidence cohorts --cohort headline_b200

Parity: scripts/evidence.py:1-253 of the reference project (same record schema, flag lists and output keys).
"""

from __future__ import annotations

import argparse
import csv
import gzip
import json
import statistics
from collections import Counter, defaultdict
from pathlib import Path
from typing import Iterable, Iterator, List, Optional

REPO = Path(__file__).resolve().parents[1]


def default_data_dir() -> Path:
    """The repo's own measurement folder, else the published data that ships with the installed baseline."""
    for cand in (REPO / "paper_data", REPO / "baseline" / "_ref" / "paper_data"):
        if (cand / "results").is_dir():
            return cand
    return REPO / "paper_data"


# flags that remove a record from every statistic
EXCLUDED = frozenset({
    "failed_execution", "smoke_only", "superseded_basis_implementation", "superseded_rng_unpinned_fidelity",
    "incomplete_training_stream", "diagnostic_probe", "environment_record",
})
# flags that remove a record from quality statistics only
QUALITY_EXCLUDED = frozenset({
    "quality_quarantined_seed_instability", "quality_not_evaluated_architecture_probe", "quality_requires_underupdate_control",
    "short_horizon_quality", "quality_overlapping_training_prefix", "quality_invalid_allocation_only_backward",
    "quality_random_label_memory_probe",
})
NEVER_COUNTED = frozenset({"failed_execution", "environment_record"})
QUALITY_METRICS = frozenset({"val_ppl", "accuracy"})
METRICS = ("peak_GiB", "time_s", "val_ppl", "accuracy", "mean_cosine_full_model", "mean_cosine_local_wrapped",
           "worst_unwrapped_cosine", "stored_MiB", "tokens_per_s")
PROTOCOL_KEYS = ("tag", "cohort", "model", "bs", "bs_per_rank", "seq", "steps", "steps_ran", "steps_measured", "world_size", "dtype",
                 "amp", "eight_bit", "dataset", "attn_impl", "attn_requested", "optimizer_actual", "optimizer_state_dtype", "alloc_conf")
METHOD_KEYS = ("stacr_cfg", "rank", "rank_used", "residual_budget", "selector", "n_checkpointed_blocks", "n_wrapped_layers",
               "n_offloaded_blocks", "n_frozen_params", "ckpt_mode")
PLATFORMS = ("b200", "rtx5090", "rtx5090_cluster", "a100", "h100")


def canonical(value) -> str:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=False, allow_nan=False)


def _reject_constant(name):
    raise ValueError("Non-finite JSON: " + name)


def read_jsonl(path: Path) -> Iterator[dict]:
    opener = gzip.open if path.suffix == ".gz" else open
    with opener(path, "rt", encoding="utf-8") as fh:
        for line in fh:
            if line.strip():
                yield json.loads(line, parse_constant=_reject_constant)


def load(data: Optional[Path] = None) -> List[dict]:
    return list(read_jsonl(Path(data or default_data_dir()) / "results" / "records.jsonl"))


def select_records(records: Iterable[dict], experiment: Optional[str] = None, platform: Optional[str] = None) -> List[dict]:
    records = list(records)
    if experiment is not None and not any(experiment in r["experiments"] for r in records):
        raise ValueError("Unknown experiment: " + experiment)
    return [r for r in records if (platform is None or r["platform"] == platform) and (experiment is None or experiment in r["experiments"])]


def _method_of(row: dict) -> str:
    for key in ("method", "variant", "comparator"):
        if key in row:
            return row[key]
    return "unknown"


def _metric_stats(group: List[dict], metric: str, include_flagged: bool) -> Optional[dict]:
    per_seed = defaultdict(list)
    for rec in group:
        flags = set(rec["flags"])
        if flags & NEVER_COUNTED:
            continue
        if not include_flagged and (flags & EXCLUDED or (metric in QUALITY_METRICS and flags & QUALITY_EXCLUDED)):
            continue
        value = rec["row"].get(metric)
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            per_seed[rec["row"].get("seed", rec["record_id"])].append(float(value))
    if not per_seed:
        return None
    values = [statistics.mean(v) for v in per_seed.values()]
    return {"mean": statistics.mean(values), "std": statistics.stdev(values) if len(values) > 1 else None,
            "n_independent_seeds_or_unseeded_runs": len(values), "n_runs": sum(len(v) for v in per_seed.values()),
            "min": min(values), "max": max(values)}


def summarize(records: Iterable[dict], experiment: Optional[str] = None, include_flagged: bool = False) -> List[dict]:
    groups = defaultdict(list)
    for rec in records:
        row = rec["row"]
        key = canonical([rec["platform"], experiment or rec["experiments"][0], {k: row[k] for k in PROTOCOL_KEYS if k in row},
                         _method_of(row), {k: row[k] for k in METHOD_KEYS if k in row}])
        groups[key].append(rec)
    out = []
    for key in sorted(groups):
        group = groups[key]
        platform, series, protocol, method, method_config = json.loads(key)
        entry = {"platform": platform, "experiment": series, "protocol": protocol, "method": method, "method_config": method_config,
                 "records": len(group), "seeds": sorted({r["row"]["seed"] for r in group if isinstance(r["row"].get("seed"), int)}),
                 "flags": dict(Counter(f for r in group for f in r["flags"])), "metrics": {}}
        for metric in METRICS:
            stats = _metric_stats(group, metric, include_flagged)
            if stats:
                entry["metrics"][metric] = stats
        out.append(entry)
    return out


def _write(result, path: Path, flatten: bool) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    if flatten and path.suffix.lower() == ".csv":
        rows = []
        for entry in result:
            flat = {k: canonical(v) if isinstance(v, (dict, list)) else v for k, v in entry.items() if k != "metrics"}
            for metric, stats in entry["metrics"].items():
                flat.update({f"{metric}_{k}": v for k, v in stats.items()})
            rows.append(flat)
        with path.open("w", encoding="utf-8", newline="") as fh:
            writer = csv.DictWriter(fh, fieldnames=sorted({k for r in rows for k in r}))
            writer.writeheader()
            writer.writerows(rows)
    else:
        path.write_text(json.dumps(result, indent=2, ensure_ascii=False, allow_nan=False) + "\n", encoding="utf-8")


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--data", type=Path, default=None)
    sub = parser.add_subparsers(dest="command", required=True)
    sub.add_parser("list", help="experiment names with record counts")
    p = sub.add_parser("cohorts", help="recompute cohort statistics and check them against the published tables")
    p.add_argument("--cohort")
    p.add_argument("--output", type=Path)
    p = sub.add_parser("summary", help="aggregate runs that share hardware and protocol")
    p.add_argument("--experiment")
    p.add_argument("--platform", choices=PLATFORMS)
    p.add_argument("--include-flagged", action="store_true", help="keep diagnostic or excluded measurements (flags stay visible)")
    p.add_argument("--output", type=Path, help="JSON, or CSV when the name ends in .csv")
    args = parser.parse_args(argv)
    data = args.data or default_data_dir()
    if args.command == "cohorts":
        from .cohorts import recompute
        result = recompute(data, args.cohort)
    elif args.command == "list":
        counts = Counter(name for rec in load(data) for name in rec["experiments"])
        result = [{"experiment": name, "records": n} for name, n in sorted(counts.items())]
    else:
        result = summarize(select_records(load(data), args.experiment, args.platform), args.experiment, args.include_flagged)
    output = getattr(args, "output", None)
    if output:
        _write(result, output, flatten=args.command == "summary")
        print(str(output))
    else:
        print(json.dumps(result, indent=2, ensure_ascii=False, allow_nan=False))
    if args.command == "cohorts" and not result["all_checks_passed"]:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
