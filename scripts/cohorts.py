"""Seed means, sample standard deviations and paired per-seed comparisons for each measurement cohort.

Input: ``results/cohorts.csv`` with columns ``cohort, method, seed, accuracy, ppl, peak_gib, time_s, tokens_per_s,
cosine, timing_excluded``.  Per method, repeated executions of one seed are averaged before the across-seed
statistics; rows marked ``timing_excluded`` do not enter ``time_s``.  Paired comparisons are formed on the seeds
that both methods ran.  Every published table cell that can be derived from the cohort file is then recomputed
and compared with the table at the table's own rounding (half a unit in the last printed digit); a table that is
not present next to the data is skipped.

Parity: scripts/cohorts.py:1-285 of the reference project.
"""

from __future__ import annotations

import csv
import math
import statistics
from collections import defaultdict
from pathlib import Path
from typing import Callable, Dict, List, Optional

VALUE_COLUMNS = ("accuracy", "ppl", "peak_gib", "time_s", "tokens_per_s", "cosine")
PAIRED_COLUMNS = ("accuracy", "ppl", "peak_gib", "time_s", "tokens_per_s")

# cohort-specific pairings that are not "everything against baseline"
EXTRA_PAIRS = {"galore_composition": [("galore_alone", "stacr_galore"), ("galore_alone", "turbofast_galore")]}
REPLACED_PAIRS = {"matched_bytes": [(f"{family}_none_r{rank}", f"{family}_topk") for family, rank in
                                    (("bert_base_3ep", 139), ("bert_large_3ep", 182), ("gpt2_large_10k", 144), ("gpt2_xl_5k", 178))]}


def _finite(text) -> Optional[float]:
    try:
        v = float(text)
    except (TypeError, ValueError):
        return None
    return v if math.isfinite(v) else None


def _describe(values) -> Optional[dict]:
    values = list(values)
    if not values:
        return None
    return {"mean": statistics.mean(values), "std": statistics.stdev(values) if len(values) > 1 else None, "n": len(values)}


def read_cohorts(data: Path) -> Dict[str, List[dict]]:
    cohorts = defaultdict(list)
    with (Path(data) / "results" / "cohorts.csv").open(encoding="utf-8", newline="") as fh:
        for line in csv.DictReader(fh):
            sample = {"method": line["method"], "seed": int(line["seed"]), "timing_excluded": line["timing_excluded"].strip().lower() == "true"}
            for col in VALUE_COLUMNS:
                v = _finite(line.get(col))
                if v is not None:
                    sample[col] = v
            cohorts[line["cohort"]].append(sample)
    return cohorts


def _by_method_seed(samples):
    table = defaultdict(lambda: defaultdict(list))
    for s in samples:
        table[s["method"]][s["seed"]].append(s)
    return table


def method_summary(samples) -> dict:
    out = {}
    for method, seeds in _by_method_seed(samples).items():
        metrics = {}
        for col in VALUE_COLUMNS:
            seed_means = []
            for rows in seeds.values():
                vals = [r[col] for r in rows if col in r and not (col == "time_s" and r["timing_excluded"])]
                if vals:
                    seed_means.append(statistics.mean(vals))
            stats = _describe(seed_means)
            if stats:
                metrics[col] = stats
        out[method] = {"seeds": sorted(seeds), "metrics": metrics}
    return out


def paired(samples, reference: str, method: str) -> dict:
    table = _by_method_seed(samples)
    common = sorted(set(table[reference]) & set(table[method]))
    acc = defaultdict(list)
    for seed in common:
        ref_rows, new_rows = table[reference][seed], table[method][seed]
        for col in PAIRED_COLUMNS:
            if col == "time_s" and any(r["timing_excluded"] for r in ref_rows + new_rows):
                continue
            ref = [r[col] for r in ref_rows if col in r]
            new = [r[col] for r in new_rows if col in r]
            if not ref or not new:
                continue
            b, v = statistics.mean(ref), statistics.mean(new)
            acc["reference_" + col].append(b)
            acc["method_" + col].append(v)
            acc[col + "_difference"].append(v - b)
            if b:
                acc[col + "_ratio"].append(v / b)
                acc[col + "_delta_pct"].append(100.0 * (v / b - 1.0))
    return {"reference": reference, "method": method, "paired_seeds": common, "metrics": {k: _describe(v) for k, v in acc.items()}}


def _pairs_for(name: str, methods: dict):
    if name in REPLACED_PAIRS:
        return list(REPLACED_PAIRS[name])
    pairs = [("baseline", m) for m in methods if m != "baseline"] if "baseline" in methods else []
    return pairs + EXTRA_PAIRS.get(name, [])


class _TableChecker:
    """Compares recomputed values with cells of the published CSV tables at the printed precision."""

    def __init__(self, data: Path):
        self.data, self.checks, self._tables = Path(data), [], {}

    def _table(self, name: str):
        if name not in self._tables:
            path = self.data / name
            if not path.is_file():
                self._tables[name] = None
            else:
                with path.open(encoding="utf-8-sig", newline="") as fh:
                    self._tables[name] = list(csv.DictReader(fh))
        return self._tables[name]

    def __call__(self, cohort: str, table: str, row_label: str, column: str, computed) -> None:
        rows = self._table(table)
        if rows is None:
            return
        row = next((r for r in rows if next(iter(r.values())) == row_label), None)
        if row is None or not row.get(column):
            return
        printed = row[column].split()[0]
        decimals = len(printed.partition(".")[2])
        tol = 0.500001 * 10.0 ** (-decimals)
        expected = float(printed)
        self.checks.append({"cohort": cohort, "table": table, "row": row_label, "column": column, "expected": expected, "computed": computed,
                            "rounding_tolerance": tol, "passed": computed is not None and abs(computed - expected) <= tol})


def _stat(result: dict, method: str, metric: str, which: str):
    try:
        return result["methods"][method]["metrics"][metric][which]
    except KeyError:
        return None


def _check_pythia(result, check):
    for method, label in (("baseline", "10k baseline 5-seed"), ("stacr", "10k STAC-R 5-seed"), ("turbo_fast", "10k Turbo-fast 5-seed")):
        check("pythia_10k", "pythia_longhorizon.csv", label, "ppl", _stat(result, method, "ppl", "mean"))
        if method != "turbo_fast":
            check("pythia_10k", "pythia_longhorizon.csv", label, "ppl_std", _stat(result, method, "ppl", "std"))


def _check_galore(result, check):
    columns = (("ppl_mean", "ppl", "mean"), ("ppl_std", "ppl", "std"), ("peak_gib", "peak_gib", "mean"), ("time_s", "time_s", "mean"))
    for method, label in (("baseline", "baseline"), ("galore_alone", "GaLore"), ("stacr_galore", "STAC-R + GaLore"), ("turbofast_galore", "Turbo-fast + GaLore")):
        for column, metric, which in columns:
            check("galore_composition", "composition.csv", label, column, _stat(result, method, metric, which))
    marginal = (("ppl_mean", "ppl_difference", "mean"), ("ppl_std", "ppl_difference", "std"), ("peak_gib", "peak_gib_difference", "mean"),
                ("time_s", "time_s_difference", "mean"), ("peak_delta_pct", "peak_gib_delta_pct", "mean"))
    for pair in result["paired_comparisons"]:
        if pair["reference"] != "galore_alone":
            continue
        label = "STAC-R marginal over GaLore" if pair["method"] == "stacr_galore" else "Turbo-fast marginal over GaLore"
        for column, metric, which in marginal:
            stats = pair["metrics"].get(metric)
            check("galore_composition", "composition.csv", label, column, stats[which] if stats else None)


def _check_bert(result, check):
    if not result["paired_comparisons"]:
        return
    pair = result["paired_comparisons"][0]
    for column, metric in (("memory_delta_pct", "peak_gib_delta_pct"), ("time_x", "time_s_ratio"), ("quality_delta", "accuracy_difference")):
        stats = pair["metrics"].get(metric)
        check("bert_sst2", "quality_cost_summary.csv", "BERT-base SST-2", column, stats["mean"] if stats else None)


def _check_matched(result, check):
    labels = {"bert_base_3ep_topk": "BERT-base SST-2", "bert_large_3ep_topk": "BERT-large SST-2", "gpt2_large_10k_topk": "GPT-2 Large WT103",
              "gpt2_xl_5k_topk": "GPT-2 XL WT103"}
    for pair in result["paired_comparisons"]:
        label = labels.get(pair["method"])
        if label is None:
            continue
        for column, metric in (("hybrid_tok_s", "method_tokens_per_s"), ("pure_lr_tok_s", "reference_tokens_per_s"), ("gain_pct", "tokens_per_s_delta_pct")):
            stats = pair["metrics"].get(metric)
            check("matched_bytes", "matched_budget_throughput.csv", label, column, stats["mean"] if stats else None)
        check("matched_bytes", "matched_budget_throughput.csv", label, "seeds", len(pair["paired_seeds"]))


def _check_gamma(result, check):
    """Residual gain: epsilon = (1-cos)/(1+cos); gamma = 1 - (eps_on/eps_off)^2 for each rank with and without the residual."""
    derived = []
    for rank in (8, 32, 128, 307):
        on, off = _stat(result, f"rank{rank}_block_sparse", "cosine", "mean"), _stat(result, f"rank{rank}_none", "cosine", "mean")
        if on is None or off is None:
            continue
        eps_on, eps_off = (1 - on) / (1 + on), (1 - off) / (1 + off)
        row = {"rank": rank, "cosine_on": on, "cosine_off": off, "epsilon_on": eps_on, "gamma_epsilon": 1 - (eps_on / eps_off) ** 2}
        derived.append(row)
        for column in ("cosine_on", "cosine_off", "epsilon_on", "gamma_epsilon"):
            check("residual_gamma", "residual_gamma.csv", str(rank), column, row[column])
    result["derived_rows"] = derived


def _check_headline_b200(result, check):
    """This build's own cohort: throughput of the sm_100a path and of the reference arm on the same B200."""
    for method, label in (("baseline", "reference arm"), ("stacr_b200", "stacr_b200")):
        check("headline_b200", "b200_headline.csv", label, "tokens_per_s", _stat(result, method, "tokens_per_s", "mean"))
        check("headline_b200", "b200_headline.csv", label, "peak_gib", _stat(result, method, "peak_gib", "mean"))


COHORT_CHECKS: Dict[str, Callable] = {"pythia_10k": _check_pythia, "galore_composition": _check_galore, "bert_sst2": _check_bert,
                                      "matched_bytes": _check_matched, "residual_gamma": _check_gamma, "headline_b200": _check_headline_b200}


def recompute(data, selected: Optional[str] = None) -> dict:
    data = Path(data)
    cohorts = read_cohorts(data)
    if selected and selected not in cohorts:
        raise ValueError("Unknown recomputable cohort: " + selected)
    output = {}
    for name, samples in cohorts.items():
        if selected and name != selected:
            continue
        methods = method_summary(samples)
        output[name] = {"methods": methods, "paired_comparisons": [paired(samples, a, b) for a, b in _pairs_for(name, methods)]}
    checker = _TableChecker(data)
    for name, fn in COHORT_CHECKS.items():
        if name in output:
            fn(output[name], checker)
    return {"cohorts": output, "published_cell_checks": checker.checks, "all_checks_passed": all(c["passed"] for c in checker.checks)}
