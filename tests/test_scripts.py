"""Evidence tooling: record summaries, cohort recomputation against table cells, table rendering, gradient-bound probe."""

import csv
import json
import math

import pytest
import torch

from scripts import aggregate_results, cohorts, evidence, make_tables, records, theorem_probe


def _record(rid, platform, exp, flags, **row):
    return {"record_id": rid, "platform": platform, "experiments": [exp], "flags": flags, "row": row}


def _write_records(tmp_path, recs):
    (tmp_path / "results").mkdir(parents=True, exist_ok=True)
    with (tmp_path / "results" / "records.jsonl").open("w") as fh:
        for r in recs:
            fh.write(json.dumps(r) + "\n")


def test_summary_averages_repeats_per_seed_and_honours_flags(tmp_path):
    recs = [
        _record("a", "b200", "headline", [], method="stacr", model="m", seed=1, tokens_per_s=100.0, val_ppl=20.0),
        _record("b", "b200", "headline", [], method="stacr", model="m", seed=1, tokens_per_s=200.0, val_ppl=22.0),  # repeat of seed 1
        _record("c", "b200", "headline", [], method="stacr", model="m", seed=2, tokens_per_s=300.0, val_ppl=24.0),
        _record("d", "b200", "headline", ["smoke_only"], method="stacr", model="m", seed=3, tokens_per_s=9e9),
        _record("e", "b200", "headline", ["short_horizon_quality"], method="stacr", model="m", seed=4, tokens_per_s=500.0, val_ppl=1e9),
        _record("f", "h100", "headline", ["failed_execution"], method="stacr", model="m", seed=5, tokens_per_s=1.0),
    ]
    _write_records(tmp_path, recs)
    loaded = evidence.load(tmp_path)
    out = evidence.summarize(evidence.select_records(loaded, "headline", "b200"), "headline")
    assert len(out) == 1
    tps = out[0]["metrics"]["tokens_per_s"]
    assert tps["n_independent_seeds_or_unseeded_runs"] == 3 and tps["n_runs"] == 4  # seeds 1, 2, 4; the smoke run is excluded
    assert tps["mean"] == pytest.approx((150.0 + 300.0 + 500.0) / 3)
    ppl = out[0]["metrics"]["val_ppl"]
    assert ppl["n_independent_seeds_or_unseeded_runs"] == 2 and ppl["mean"] == pytest.approx(22.5)  # quality flag removes seed 4
    flagged = evidence.summarize(evidence.select_records(loaded, "headline", "b200"), "headline", include_flagged=True)
    assert flagged[0]["metrics"]["tokens_per_s"]["max"] == 9e9
    all_platforms = evidence.summarize(loaded, "headline", include_flagged=True)
    h100 = next(e for e in all_platforms if e["platform"] == "h100")
    assert h100["metrics"] == {}  # a failed execution is never counted
    with pytest.raises(ValueError):
        evidence.select_records(loaded, "nonexistent")


def test_records_reject_nonfinite_json(tmp_path):
    (tmp_path / "results").mkdir()
    (tmp_path / "results" / "records.jsonl").write_text('{"record_id":"x","platform":"b200","experiments":["e"],"flags":[],"row":{"v":NaN}}\n')
    with pytest.raises(ValueError):
        evidence.load(tmp_path)


def test_cohort_statistics_pairs_and_table_check(tmp_path):
    (tmp_path / "results").mkdir()
    rows = [
        ("bert_sst2", "baseline", 1, 90.0, "", 2.0, 100.0, "", "", "false"),
        ("bert_sst2", "baseline", 2, 92.0, "", 2.0, 110.0, "", "", "false"),
        ("bert_sst2", "full", 1, 91.0, "", 1.0, 200.0, "", "", "false"),
        ("bert_sst2", "full", 2, 91.0, "", 1.5, 999.0, "", "", "true"),   # timing of seed 2 is excluded
        ("bert_sst2", "full", 3, 80.0, "", 1.0, 150.0, "", "", "false"),  # unpaired seed
    ]
    with (tmp_path / "results" / "cohorts.csv").open("w", newline="") as fh:
        w = csv.writer(fh)
        w.writerow(cohorts.VALUE_COLUMNS and ["cohort", "method", "seed", "accuracy", "ppl", "peak_gib", "time_s", "tokens_per_s", "cosine", "timing_excluded"])
        w.writerows(rows)
    (tmp_path / "quality_cost_summary.csv").write_text("task,memory_delta_pct,time_x,quality_delta\nBERT-base SST-2,-37.5,2.00,0.0\n")
    out = cohorts.recompute(tmp_path)
    pair = out["cohorts"]["bert_sst2"]["paired_comparisons"][0]
    assert pair["paired_seeds"] == [1, 2]
    assert pair["metrics"]["peak_gib_delta_pct"]["mean"] == pytest.approx((-50.0 - 25.0) / 2)
    assert pair["metrics"]["time_s_ratio"]["n"] == 1 and pair["metrics"]["time_s_ratio"]["mean"] == pytest.approx(2.0)
    assert out["cohorts"]["bert_sst2"]["methods"]["full"]["metrics"]["time_s"]["n"] == 2
    assert out["all_checks_passed"] and len(out["published_cell_checks"]) == 3
    (tmp_path / "quality_cost_summary.csv").write_text("task,memory_delta_pct,time_x,quality_delta\nBERT-base SST-2,-30.0,2.00,0.0\n")
    assert not cohorts.recompute(tmp_path)["all_checks_passed"]
    with pytest.raises(ValueError):
        cohorts.recompute(tmp_path, "no_such_cohort")


def test_repo_measurements_are_self_consistent():
    out = cohorts.recompute(evidence.REPO / "paper_data", "headline_b200")
    assert out["all_checks_passed"] and out["published_cell_checks"]
    ratio = out["cohorts"]["headline_b200"]["paired_comparisons"][0]["metrics"]["tokens_per_s_ratio"]["mean"]
    assert ratio > 1.0


def test_bench_line_to_record_is_idempotent(tmp_path):
    line = {"metric": "tokens_per_second", "value": 1000.0, "n_gpus": 1, "steps": 4, "ms_per_step": 10.0, "dtype": "bf16", "impl": "reference",
            "config": {"model": "tiny", "global_batch": 2, "seq_len": 8}, "memory": {"peak_allocated_gb": 1.0}}
    src = tmp_path / "line.json"
    src.write_text("NCCL banner\n" + json.dumps(line) + "\n")
    assert records.add([src], tmp_path / "data", "b200", "c", "e") == 1
    assert records.add([src], tmp_path / "data", "b200", "c", "e") == 0
    rec = evidence.load(tmp_path / "data")[0]
    assert rec["row"]["method"] == "baseline" and rec["row"]["peak_GiB"] == pytest.approx(1e9 / 2 ** 30)


def test_tables_and_aggregation(tmp_path):
    (tmp_path / "a.csv").write_text("name,value\nx_1,50%\n")
    (tmp_path / "b.csv").write_text("name,other\ny,3\n")
    (tmp_path / "main_results.csv").write_text("name\nold\n")
    out = tmp_path / "all.csv"
    aggregate_results.main(["--input", str(tmp_path), "--output", str(out)])
    with out.open() as fh:
        rows = list(csv.DictReader(fh))
    assert [r["name"] for r in rows] == ["x_1", "y"] and set(rows[0]) == {"name", "value", "other"}
    tex = make_tables.csv_to_latex(tmp_path / "a.csv")
    assert r"x\_1 & 50\%" in tex and tex.startswith(r"\begin{tabular}{ll}")
    make_tables.main(["--input", str(tmp_path), "--output", str(tmp_path / "tex")])
    assert (tmp_path / "tex" / "a.tex").is_file()
    assert make_tables.escape_latex("a&b~") == r"a\&b\textasciitilde{}"


def test_theorem_probe_single_and_paired(tmp_path):
    from stacr_b200 import apply_stacr
    from stacr_b200.models import build_model

    torch.manual_seed(0)
    dense = build_model("gpt-tiny")
    torch.save({"model": dense.state_dict()}, tmp_path / "dense.pt")
    report = theorem_probe.main(["--checkpoint", str(tmp_path / "dense.pt"), "--model", "gpt-tiny", "--rank", "4", "--batch-size", "4", "--max-length", "32"])
    assert report["mode"] == "single" and report["summary"]["num_layers"] > 0
    assert report["summary"]["projection_bound_violations"] == 0
    assert report["summary"]["grad_vectors_match"] == report["summary"]["num_layers"]
    for layer in report["per_layer"].values():
        # with an exact projector the residual gradient is orthogonal to the kept part: cos^2 = 1 - p
        assert layer["cos_proj_observed"] == pytest.approx(math.sqrt(1 - layer["p"]), abs=1e-3)
        assert 0.0 <= layer["EV_A"] <= 1.0 and layer["kappa_G"] >= 1.0 - 1e-4
    wrapped = build_model("gpt-tiny")
    wrapped.load_state_dict(dense.state_dict())
    apply_stacr(wrapped, rank=4, surface="mlp+attention", min_features=8, residual_mode="block_sparse")
    batch = theorem_probe.build_batch("synthetic", wrapped, 4, 32, 0)
    wrapped.train()
    wrapped(**batch).loss.backward()
    torch.save({"model": wrapped.state_dict()}, tmp_path / "wrapped.pt")
    paired = theorem_probe.main(["--baseline-checkpoint", str(tmp_path / "dense.pt"), "--stacr-checkpoint", str(tmp_path / "wrapped.pt"), "--model", "gpt-tiny",
                                 "--rank", "4", "--batch-size", "4", "--max-length", "32", "--output", str(tmp_path / "probe.json")])
    assert paired["mode"] == "paired" and "mean_cos_full_observed" in paired["summary"]
    assert json.loads((tmp_path / "probe.json").read_text())["metadata"]["comparison_scope"] == "different_trained_checkpoints"
    with pytest.raises(SystemExit):
        theorem_probe.main(["--model", "gpt-tiny"])
    assert theorem_probe.cosine_bound(1.5) is None and theorem_probe.finite_json({"a": float("nan")}) == {"a": None}
