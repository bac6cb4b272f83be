"""Service-rate calibration: how fast one Target GPU produces and one Draft GPU consumes, measured on the real path.

The reference calibrates with dedicated producer and consumer probe candidates (aspec/calibration.py:206-603).  Here
the two probes are the two EXTREME legal splits of the node, run as ordinary bounded training runs:

* the producer-heavy split (as many Target GPUs as the recipe allows) saturates the Draft ranks, so its steady-window
  rate divided by the Draft GPUs is the per-GPU consumer rate;
* the consumer-heavy split (one Target GPU) saturates that Target, so its steady-window rate is the per-GPU producer
  rate; the engines' own ``tokens / busy_seconds`` is reported beside it as a cross-check.

Both runs are end-to-end candidates in their own right, so the topology study reuses their evidence instead of running
those splits again.  A probe is a child process (``python -m aspec_b200.train_entry``) that owns the GPUs it uses and
leaves a normal run directory behind; nothing here touches a GPU itself.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import sys
import time
from typing import Callable, Dict, List, Optional, Sequence

CALIBRATION_SCHEMA_VERSION = "aspec.calibration/v1"


def bounded_run_overrides(steps: int, warmup: int) -> List[str]:
    """What turns a recipe into a short measured run: a fixed number of updates, no checkpoints, no evaluation, and a
    steady window that is required (the run fails if it cannot produce one)."""
    return [f"training.num_train_steps={int(steps)}", "training.save_interval=0", "training.save_final_checkpoint=false",
            "dataset.eval_interval=0", "debug.performance_measurement_required=true",
            f"debug.performance_warmup_steps={int(warmup)}", "debug.performance_drain_steps=0"]


def split_overrides(target_gpus: int, draft_gpus: int) -> List[str]:
    return [f"inference.inference_num_gpus={int(target_gpus)}", f"training.training_num_gpus_per_node={int(draft_gpus)}"]


def run_bounded(config_path: str, overrides: Sequence[str], run_dir: str, timeout: float = 1800.0,
                env: Optional[Dict[str, str]] = None) -> dict:
    """One bounded run in a child process; returns ``{"run": dir, "returncode": rc, "seconds": s, "evidence": {...}|None}``."""
    cmd = [sys.executable, "-m", "aspec_b200.train_entry", "--config", config_path, *overrides, f"output_dir={run_dir}"]
    t0 = time.perf_counter()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env={**os.environ, **(env or {})})
        rc, tail = proc.returncode, (proc.stderr or proc.stdout)[-800:]
    except subprocess.TimeoutExpired:
        rc, tail = -9, f"no result within {timeout:.0f} s"
    path = os.path.join(run_dir, "evidence.json")
    evidence = json.load(open(path)) if os.path.isfile(path) else None
    return {"run": run_dir, "returncode": rc, "seconds": time.perf_counter() - t0, "evidence": evidence,
            "output_tail": tail if rc else ""}


def window_of(evidence: Optional[dict]) -> dict:
    summary = (evidence or {}).get("training_summary") or {}
    return summary.get("window") or {}


def engine_rate(evidence: Optional[dict]) -> Optional[float]:
    """Median over the Target engines of tokens prefilled per second of engine busy time."""
    engines = ((evidence or {}).get("training_summary") or {}).get("engines") or []
    rates = [e["tokens"] / e["busy_seconds"] for e in engines if e.get("busy_seconds") and e.get("tokens")]
    return statistics.median(rates) if rates else None


def rates_from_probes(producer_heavy: dict, consumer_heavy: dict, splits: Dict[str, tuple]) -> dict:
    """Per-GPU service rates from the two extreme runs (``splits``: role name -> ``(target_gpus, draft_gpus)``)."""
    out = {"schema_version": CALIBRATION_SCHEMA_VERSION, "draft_tokens_per_s_per_gpu": None,
           "target_tokens_per_s_per_gpu": None, "target_engine_tokens_per_busy_s": None, "problems": []}
    w = window_of(producer_heavy.get("evidence"))
    if w.get("valid") and w.get("tokens_per_second"):
        out["draft_tokens_per_s_per_gpu"] = float(w["tokens_per_second"]) / splits["producer_heavy"][1]
    else:
        out["problems"].append(f"producer-heavy probe {producer_heavy.get('run')} has no valid steady window")
    w = window_of(consumer_heavy.get("evidence"))
    if w.get("valid") and w.get("tokens_per_second"):
        out["target_tokens_per_s_per_gpu"] = float(w["tokens_per_second"]) / splits["consumer_heavy"][0]
    else:
        out["problems"].append(f"consumer-heavy probe {consumer_heavy.get('run')} has no valid steady window")
    out["target_engine_tokens_per_busy_s"] = engine_rate(consumer_heavy.get("evidence")) or engine_rate(producer_heavy.get("evidence"))
    return out


def calibrate(config_path: str, splits: Sequence[tuple], out_dir: str, *, steps: int = 24, warmup: int = 4,
              overrides: Sequence[str] = (), runner: Callable[..., dict] = run_bounded, timeout: float = 1800.0) -> dict:
    """Run the two extreme splits of ``splits`` (a list of ``(target_gpus, draft_gpus)``) and derive the service rates.

    Returns ``{"rates": ..., "runs": {"<t>T+<d>D": run record}}``; with a single legal split there is nothing to choose
    and no probe runs."""
    splits = sorted(splits)
    if len(splits) < 2:
        return {"rates": {"schema_version": CALIBRATION_SCHEMA_VERSION, "problems": ["one legal split: nothing to calibrate"]},
                "runs": {}}
    roles = {"consumer_heavy": splits[0], "producer_heavy": splits[-1]}
    runs = {}
    for role, (t, d) in roles.items():
        name = f"{t}T+{d}D"
        runs[name] = runner(config_path, [*overrides, *split_overrides(t, d), *bounded_run_overrides(steps, warmup)],
                            os.path.join(out_dir, f"calibrate-{name}"), timeout)
    rates = rates_from_probes(runs["%dT+%dD" % roles["producer_heavy"]], runs["%dT+%dD" % roles["consumer_heavy"]], roles)
    return {"rates": rates, "runs": runs}
