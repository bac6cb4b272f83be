"""Topology study runner and calibration: logic against a simulated pipeline, and one real bounded child run
(reference: tests/test_topology_runner.py, tests/test_calibration.py)."""
import json
import os
import re

import pytest

from aspec_b200 import calibration
from aspec_b200.assets import find_asset
from aspec_b200.topology_runner import run_study


def _simulated_pipeline(target_rate, draft_rate, efficiency=0.9, fail=()):
    """A runner that behaves like a node whose Target GPUs make ``target_rate`` and Draft GPUs take ``draft_rate`` tokens/s."""
    calls = []

    def runner(config_path, overrides, run_dir, timeout):
        kv = dict(o.split("=", 1) for o in overrides)
        t, d = int(kv["inference.inference_num_gpus"]), int(kv["training.training_num_gpus_per_node"])
        calls.append((t, d))
        assert kv["debug.performance_measurement_required"] == "true" and kv["training.save_interval"] == "0"
        os.makedirs(run_dir, exist_ok=True)
        rate = min(target_rate * t, draft_rate * d) * efficiency
        ok = (t, d) not in fail
        ev = {"state": "completed", "plan_id": f"sha256:{t}-{d}", "plan": {"policy": {"target_gpus": t, "draft_gpus": d}},
              "training_summary": {"window": {"valid": ok, "tokens_per_second": rate if ok else None, "steps": 20},
                                   "ledger": {"validated": ok},
                                   "engines": [{"tokens": 1000.0 * target_rate, "busy_seconds": 1000.0}] * t}}
        json.dump(ev, open(os.path.join(run_dir, "evidence.json"), "w"))
        return {"run": run_dir, "returncode": 0 if ok else 1, "seconds": 1.0, "evidence": ev, "output_tail": ""}
    return runner, calls


def test_study_calibrates_on_the_extremes_and_picks_the_measured_best(tmp_path):
    recipe = find_asset("qwen3_8b_dspark.yaml")
    runner, calls = _simulated_pipeline(64_000.0, 96_000.0)
    res = run_study(recipe, 8, str(tmp_path), steps=24, warmup=4, top=3, runner=runner, log=None)
    assert calls[:2] == [(1, 7), (7, 1)]                                   # the two probes, then only splits not yet run
    assert len(set(calls)) == len(calls) and set(calls) >= {(5, 3), (4, 4)}
    cal = res["calibration"]
    assert cal["draft_tokens_per_s_per_gpu"] == pytest.approx(96_000 * 0.9) and cal["target_tokens_per_s_per_gpu"] == pytest.approx(64_000 * 0.9)
    assert cal["target_engine_tokens_per_busy_s"] == pytest.approx(64_000.0)
    assert res["chosen"] == "5T+3D" and res["chosen_overrides"] == ["inference.inference_num_gpus=5", "training.training_num_gpus_per_node=3"]
    assert res["ranking"][0]["median_tokens_per_s"] == pytest.approx(min(5 * 64_000, 3 * 96_000) * 0.9)
    assert all(0.99 < v < 1.01 for v in res["prediction_error"].values())
    saved = json.load(open(tmp_path / "topology-study.json"))
    assert saved["chosen"] == "5T+3D" and saved["study"]["study_id"].startswith("sha256:")


def test_a_failed_candidate_is_never_chosen_and_model_parallel_units_limit_the_splits(tmp_path):
    recipe = find_asset("qwen3_8b_dspark.yaml")
    runner, calls = _simulated_pipeline(64_000.0, 96_000.0, fail={(5, 3)})
    res = run_study(recipe, 8, str(tmp_path / "a"), runner=runner, log=None)
    assert res["chosen"] != "5T+3D" and res["runs"]["5T+3D"]["ledger_validated"] is False
    runner, calls = _simulated_pipeline(64_000.0, 96_000.0)
    res = run_study(recipe, 8, str(tmp_path / "b"), runner=runner, log=None,
                    overrides=["training.draft_context_parallel_size=2"])
    assert all(d % 2 == 0 for _, d in calls) and res["chosen"] in ("4T+4D", "6T+2D")


@pytest.mark.timeout(600)
def test_one_real_bounded_child_run_leaves_evidence_with_a_steady_window(tmp_path):
    recipe = find_asset("quickstart_tiny.yaml")
    run = calibration.run_bounded(recipe, calibration.bounded_run_overrides(steps=5, warmup=1), str(tmp_path / "probe"),
                                  timeout=500, env={"CUDA_VISIBLE_DEVICES": ""})
    assert run["returncode"] == 0, run["output_tail"]
    w = calibration.window_of(run["evidence"])
    assert w["valid"] and w["steps"] == 4 and w["tokens_per_second"] > 0
    assert run["evidence"]["training_summary"]["ledger"]["validated"]
