"""Topology study: how many of a node's GPUs should run the Target and how many the Draft.

Expert-bounded and service-rate driven, like the reference (aspec/topology.py:15-21,409-800,
aspec/calibration.py:206-603): the legal splits are enumerated from the recipe (every ``xT+yD`` whose Draft world
satisfies the recipe's CP / vocab / expert parallel divisibility), producer and consumer service rates are MEASURED
on the real path (a Target-only prefill probe and a Draft-only training probe, each a bounded run of the framework's
own engines), the balanced allocation is predicted from those rates, and the final choice is left to bounded
end-to-end runs of the top candidates, whose evidence files are ranked.

``python -m aspec_b200.topology run --config R.yaml --gpus 8 --out DIR`` does all of that automatically
(``topology_runner.run_study``); ``plan --config R.yaml`` prints the study; ``rank --runs DIR...`` ranks finished
candidate runs by their steady-window tokens/s; ``predict --target-rate X --draft-rate Y --gpus N`` applies the
balance rule to measured rates.
"""
from __future__ import annotations

import argparse
import dataclasses
import hashlib
import json
import math
import os
import statistics
import sys
from typing import Any, Dict, List, Optional, Sequence

TOPOLOGY_STUDY_SCHEMA_VERSION = "aspec.topology-study/v1"


def _identity(value: Any) -> str:
    return "sha256:" + hashlib.sha256(json.dumps(value, sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()


@dataclasses.dataclass(frozen=True)
class TopologyCandidate:
    target_gpus: int
    draft_gpus: int
    overrides: tuple
    predicted_tokens_per_s: Optional[float] = None
    bound_by: Optional[str] = None

    @property
    def name(self) -> str:
        return f"{self.target_gpus}T+{self.draft_gpus}D"


def legal_splits(total_gpus: int, *, cp: int = 1, vp: int = 1, ep: int = 1, min_target: int = 1) -> List[tuple]:
    """Every (target, draft) split whose Draft world is a multiple of the model-parallel degree."""
    unit = math.lcm(max(cp, 1), max(vp, 1), max(ep, 1))
    return [(t, total_gpus - t) for t in range(min_target, total_gpus) if (total_gpus - t) % unit == 0]


def predict(target_rate: float, draft_rate: float, target_gpus: int, draft_gpus: int, dp_efficiency: float = 1.0) -> tuple:
    """Pipeline throughput of a split from per-GPU service rates (tokens/s): the slower role bounds it."""
    produce = target_rate * target_gpus
    consume = draft_rate * draft_gpus * dp_efficiency
    return (min(produce, consume), "target" if produce < consume else "draft")


def compile_topology_study(config, total_gpus: int, *, target_rate: Optional[float] = None,
                           draft_rate: Optional[float] = None, top: int = 3) -> dict:
    t = config.training
    cp = int(getattr(t, "draft_context_parallel_size", 1) or 1)
    vp = int(getattr(t, "vocab_parallel_size", 1) or 1)
    ep = int(getattr(t, "expert_parallel_size", 1) or 1)
    cands = []
    for tg, dg in legal_splits(total_gpus, cp=cp, vp=vp, ep=ep):
        ov = (f"inference.inference_num_gpus={tg}", f"training.training_num_gpus_per_node={dg}")
        pred = bound = None
        if target_rate and draft_rate:
            pred, bound = predict(target_rate, draft_rate, tg, dg)
        cands.append(TopologyCandidate(tg, dg, ov, pred, bound))
    if target_rate and draft_rate:
        cands.sort(key=lambda c: -c.predicted_tokens_per_s)
    study = {"schema_version": TOPOLOGY_STUDY_SCHEMA_VERSION, "total_gpus": total_gpus,
             "model_parallel_unit": math.lcm(cp, vp, ep),
             "service_rates": {"target_tokens_per_s_per_gpu": target_rate, "draft_tokens_per_s_per_gpu": draft_rate},
             "probes": {"target": "bench.py --mode online --targets N (Target busy time per token)",
                        "draft": "bench.py --mode draft (resident features)"},
             "candidates": [dataclasses.asdict(c) | {"name": c.name} for c in cands],
             "end_to_end_shortlist": [c.name for c in cands[:top]]}
    study["study_id"] = _identity(study)
    return study


def load_run_rate(run_dir: str) -> Optional[dict]:
    """Steady-window rate of one finished candidate run (``evidence.json`` written by the train entry)."""
    path = os.path.join(run_dir, "evidence.json")
    if not os.path.isfile(path):
        return None
    ev = json.load(open(path))
    summary = ev.get("training_summary") or ev.get("result") or {}
    window = summary.get("window") or {}
    plan = ev.get("plan", {}).get("policy", {})
    if not window.get("tokens_per_second"):
        return None
    return {"run": run_dir, "tokens_per_second": float(window["tokens_per_second"]), "target_gpus": plan.get("target_gpus"),
            "draft_gpus": plan.get("draft_gpus"), "plan_id": ev.get("plan_id")}


def rank_runs(run_dirs: Sequence[str]) -> dict:
    by_split: Dict[str, List[float]] = {}
    skipped = []
    for d in run_dirs:
        r = load_run_rate(d)
        if r is None:
            skipped.append(d)
            continue
        by_split.setdefault(f"{r['target_gpus']}T+{r['draft_gpus']}D", []).append(r["tokens_per_second"])
    ranking = sorted(({"split": k, "runs": len(v), "median_tokens_per_s": statistics.median(v), "min": min(v), "max": max(v)}
                      for k, v in by_split.items()), key=lambda x: -x["median_tokens_per_s"])
    return {"schema_version": "aspec.topology-ranking/v1", "ranking": ranking, "skipped": skipped}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 topology", description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    plan = sub.add_parser("plan")
    plan.add_argument("--config", required=True)
    plan.add_argument("--gpus", type=int, default=8)
    plan.add_argument("--target-rate", type=float)
    plan.add_argument("--draft-rate", type=float)
    plan.add_argument("overrides", nargs="*")
    pred = sub.add_parser("predict")
    pred.add_argument("--target-rate", type=float, required=True)
    pred.add_argument("--draft-rate", type=float, required=True)
    pred.add_argument("--gpus", type=int, default=8)
    rank = sub.add_parser("rank")
    rank.add_argument("--runs", nargs="+", required=True)
    run = sub.add_parser("run", help="calibrate, run the best candidates end to end and rank them")
    run.add_argument("--config", required=True)
    run.add_argument("--gpus", type=int, default=8)
    run.add_argument("--out", required=True)
    run.add_argument("--steps", type=int, default=24)
    run.add_argument("--warmup", type=int, default=4)
    run.add_argument("--top", type=int, default=3)
    run.add_argument("--timeout", type=float, default=1800.0)
    run.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    if a.cmd == "run":
        from aspec_b200.topology_runner import run_study
        res = run_study(a.config, a.gpus, a.out, steps=a.steps, warmup=a.warmup, top=a.top, overrides=a.overrides,
                        timeout=a.timeout)
        print(json.dumps({k: res[k] for k in ("chosen", "chosen_overrides", "ranking", "calibration", "prediction_error")}, indent=2))
        return 0 if res["chosen"] else 1
    if a.cmd == "plan":
        from aspec_b200.config.train_config import load_config
        print(json.dumps(compile_topology_study(load_config(a.config, a.overrides), a.gpus, target_rate=a.target_rate,
                                                draft_rate=a.draft_rate), indent=2))
    elif a.cmd == "predict":
        rows = [{"split": f"{t}T+{d}D", "tokens_per_s": predict(a.target_rate, a.draft_rate, t, d)[0],
                 "bound_by": predict(a.target_rate, a.draft_rate, t, d)[1]} for t, d in legal_splits(a.gpus)]
        print(json.dumps(sorted(rows, key=lambda r: -r["tokens_per_s"]), indent=2))
    else:
        print(json.dumps(rank_runs(a.runs), indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
