"""Measurement-grid registry, the dry-run planner and one real CPU cell."""

import json

import pytest
import torch

from experiments.benchmarks import common
from experiments.benchmarks.__main__ import main as bench_cli
from experiments.benchmarks.registry import EXPERIMENTS


def test_registry_lists_every_grid_with_metadata():
    assert len(EXPERIMENTS) == 51
    for needed in ("sequence_length", "attention_kernels", "runtime_breakdown", "hardware_runtime", "peak_anatomy", "allocator_stability",
                   "budget_throughput", "capacity", "composed_frontier", "composition_law", "lora", "qlora", "pythia", "bert_sst2", "rate_distortion",
                   "residual_selectors", "distributed_data", "distributed_sharding"):
        assert needed in EXPERIMENTS, needed
    for name, meta in EXPERIMENTS.items():
        assert meta["description"] and meta["module"] and isinstance(meta["cells"], list), name


@pytest.mark.parametrize("name", sorted(EXPERIMENTS))
def test_every_grid_plans_without_touching_a_model(name, tmp_path, monkeypatch):
    def boom(*a, **k):
        raise AssertionError("the planner must not build a model")

    monkeypatch.setattr(common, "load_model", boom)
    out = tmp_path / "plan.json"
    assert bench_cli(["run", name, "--dry-run", "--plan-output", str(out)]) == 0
    plan = json.loads(out.read_text())
    assert plan["experiment"] == name and plan["n_cells"] == len(plan["cells"]) > 0
    assert all("method" in c or "comparator" in c or "arm" in c for c in plan["cells"])


def test_planner_overrides_and_cohort_filter(tmp_path, capsys):
    assert bench_cli(["run", "pythia", "--dry-run", "--steps", "7", "--seeds", "5", "--batch-size", "3"]) == 0
    plan = json.loads(capsys.readouterr().out)
    assert {c["seed"] for c in plan["cells"]} == {5} and all(c["steps"] == 7 and c["bs"] == 3 for c in plan["cells"])
    before = len(plan["cells"])
    assert bench_cli(["run", "pythia", "--dry-run", "--cohort", "baseline"]) == 0
    filtered = json.loads(capsys.readouterr().out)
    assert 0 < filtered["n_cells"] < before * 3 and all("baseline" in c["method"] for c in filtered["cells"])
    assert bench_cli(["list"]) == 0 and "sequence_length" in capsys.readouterr().out
    assert bench_cli(["run", "distributed_data"]) == 2       # multi-process grid: prints its launch line
    with pytest.raises(SystemExit):
        bench_cli(["run", "not_a_grid", "--dry-run"])


def test_one_real_cell_on_cpu_reports_ledger_and_throughput():
    common.set_recorder(None)
    row = common.run_config("stacr", seed=1, model_id="gpt-tiny", bs=2, seq=32, steps=4, measure_from=1, device="cpu", eval_batches=1, eight_bit=False,
                            stacr_cfg={"rank": 4, "residual_budget": 0.01, "surface": "mlp", "min_features": 8}, baseline_peak_bytes=1 << 30)
    assert row["status"] == "ok" and row["n_wrapped_layers"] > 0 and row["steps_measured"] == 3
    assert row["tokens_per_s"] > 0 and row["validation_ppl"] > 1.0
    ledger = common.SSPLedger([])
    assert ledger.report(1 << 30) == {}                       # nothing probed: no prediction
    assert 0 < row["ssp"]["payload_bytes"] < row["ssp"]["wrapped_bytes"] and row["ssp"]["ssp"] > 0
    dense = common.run_config("baseline", seed=1, model_id="gpt-tiny", bs=2, seq=32, steps=2, measure_from=0, device="cpu", eval_batches=0, eight_bit=False)
    assert dense["n_wrapped_layers"] == 0 and dense["validation_ppl"] is None


def test_emit_appends_json_lines(tmp_path):
    path = tmp_path / "rows.jsonl"
    common.emit({"a": 1, "t": torch.tensor(2.0)}, path)
    common.emit({"a": 2}, path)
    rows = [json.loads(l) for l in path.read_text().splitlines()]
    assert [r["a"] for r in rows] == [1, 2]
