"""The benchmark entry point's output contract, on CPU with tiny shapes (not a valid measurement, only the format)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REQUIRED = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
            "dtype", "data", "config", "e2e", "gpu_launches", "clocks"}


def _run(cmd, env=None):
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600, env={**os.environ, **(env or {})})
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


@pytest.mark.timeout(600)
def test_single_process_line_has_every_key_and_an_end_to_end_number():
    res = _run([sys.executable, "bench.py", "--small", "--steps", "2", "--warmup", "1"], {"CUDA_VISIBLE_DEVICES": ""})
    assert REQUIRED <= set(res)
    assert res["n_gpus"] == 1 and res["steps"] == 2 and res["warmup"] == 1 and res["higher_is_better"] is True
    assert res["value"] > 0 and res["ms_per_step"] > 0
    e2e = res["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] >= 0 and e2e["d2h_bytes_per_step"] > 0
    assert res["config"]["parallelism"] == "dp1" and "l2_policy" in res["config"]


@pytest.mark.timeout(900)
def test_two_ranks_under_torchrun_print_one_line_with_the_aggregate():
    res = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                "--master-port", str(29600 + os.getpid() % 300), "bench.py", "--gpus", "2", "--small", "--steps", "1", "--warmup", "1",
                "--no-e2e"], {"CUDA_VISIBLE_DEVICES": ""})
    assert res["n_gpus"] == 2 and res["config"]["parallelism"] == "dp2+sharded_optimizer" and res["config"]["global_batch"] == 32
    assert res["vs_baseline"] is None and "length sequence of the 1-GPU run" in res["config"]["dp_balance"]


def test_online_split_search_runs_the_predicted_split_and_keeps_the_measured_best(monkeypatch):
    import argparse
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    asked = []

    rate = {"target": 40e3}

    def fake_child(args, targets=0):
        t = targets or args.gpus // 2
        d = args.gpus - t
        asked.append(t)
        value = min(rate["target"] * t, 96e3 * 0.8 * d) * 0.95
        return {"value": value, "targets": t, "drafts": d, "ledger_validated": True,
                "target_tokens": [rate["target"] * 20] * t, "target_busy_seconds": [20.0] * t}
    monkeypatch.setattr(bench, "online_child", fake_child)
    # a slow Target: five Target GPUs beat four even with ring-fed Drafts at 0.8 of their resident rate
    out = bench.online_with_split_search(argparse.Namespace(gpus=8, targets=0), draft_rate=96e3)
    assert asked == [4, 5] and out["targets"] == 5 and out["drafts"] == 3
    assert [r["split"] for r in out["split_search"]["runs"]] == ["4T+4D", "5T+3D"]
    assert out["split_search"]["predicted"][0]["split"] == "5T+3D"
    # the measured B200 rates: 4T+4D stays, no second run
    asked.clear()
    rate["target"] = 68.5e3
    out = bench.online_with_split_search(argparse.Namespace(gpus=8, targets=0), draft_rate=97.8e3)
    assert asked == [4] and out["targets"] == 4 and out["split_search"]["predicted"][0]["split"] == "4T+4D"
    asked.clear()
    out = bench.online_with_split_search(argparse.Namespace(gpus=4, targets=0), draft_rate=96e3)
    assert asked == [2] and out["targets"] == 2                       # 2T+2D is already the balanced split of four GPUs
