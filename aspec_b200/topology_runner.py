"""Automatic topology study: calibrate, predict, run the best candidates end to end, rank them by evidence.

``run_study`` is what ``python -m aspec_b200.topology run --config R.yaml --gpus 8 --out DIR`` executes (the reference's
counterpart: aspec/topology_runner.py, which schedules probe and candidate trials on a Ray cluster).  Every trial is a
bounded child run of the ordinary train entry in its own run directory, so each carries its own plan, evidence and work
ledger; the study only reads those files.  Steps:

1. the legal splits come from the recipe (``topology.legal_splits``: the Draft world must be a multiple of the
   context / vocab / expert parallel unit);
2. the two extreme splits are run first and give the per-GPU producer and consumer service rates
   (``calibration.calibrate``);
3. the balance rule predicts every split's rate; the ``top`` predicted splits that have not run yet are run;
4. all finished runs are ranked by their measured steady-window tokens/s; the winner's overrides are the answer.

Nothing is extrapolated into the answer: a split is only chosen if it ran and its ledger validated.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Optional, Sequence

from aspec_b200 import calibration
from aspec_b200.topology import compile_topology_study, legal_splits, rank_runs

STUDY_RESULT_SCHEMA_VERSION = "aspec.topology-study-result/v1"


def _ledger_ok(run: dict) -> bool:
    ev = run.get("evidence") or {}
    ledger = (ev.get("training_summary") or {}).get("ledger") or {}
    return run.get("returncode") == 0 and bool(ledger.get("validated", False))


def run_study(config_path: str, total_gpus: int, out_dir: str, *, steps: int = 24, warmup: int = 4, top: int = 3,
              overrides: Sequence[str] = (), runner: Callable[..., dict] = calibration.run_bounded,
              timeout: float = 1800.0, log: Optional[Callable[[str], None]] = print) -> dict:
    from aspec_b200.config.train_config import load_config
    say = log or (lambda _m: None)
    os.makedirs(out_dir, exist_ok=True)
    config = load_config(config_path, list(overrides))
    t = config.training
    splits = legal_splits(total_gpus, cp=int(getattr(t, "draft_context_parallel_size", 1) or 1),
                          vp=int(getattr(t, "vocab_parallel_size", 1) or 1), ep=int(getattr(t, "expert_parallel_size", 1) or 1))
    if not splits:
        raise ValueError(f"no split of {total_gpus} GPUs satisfies the recipe's model-parallel degrees")
    say(f"[topology] {len(splits)} legal splits of {total_gpus} GPUs; calibrating on the extremes")
    cal = calibration.calibrate(config_path, splits, out_dir, steps=steps, warmup=warmup, overrides=overrides,
                                runner=runner, timeout=timeout)
    rates = cal["rates"]
    study = compile_topology_study(config, total_gpus, target_rate=rates.get("target_tokens_per_s_per_gpu"),
                                   draft_rate=rates.get("draft_tokens_per_s_per_gpu"), top=top)
    runs = dict(cal["runs"])
    bound = calibration.bounded_run_overrides(steps, warmup)
    for name in study["end_to_end_shortlist"]:
        if name in runs:
            continue
        cand = next(c for c in study["candidates"] if c["name"] == name)
        say(f"[topology] running candidate {name} (predicted {cand['predicted_tokens_per_s']})")
        runs[name] = runner(config_path, [*overrides, *cand["overrides"], *bound], os.path.join(out_dir, f"candidate-{name}"), timeout)
    if len(splits) == 1 and not runs:                # nothing to choose between: still measure the one split
        tg, dg = splits[0]
        runs[f"{tg}T+{dg}D"] = runner(config_path, [*overrides, *calibration.split_overrides(tg, dg), *bound],
                                      os.path.join(out_dir, f"candidate-{tg}T+{dg}D"), timeout)
    good = {n: r for n, r in runs.items() if _ledger_ok(r)}
    ranking = rank_runs([r["run"] for r in good.values()])
    winner = ranking["ranking"][0]["split"] if ranking["ranking"] else None
    chosen = next((c for c in study["candidates"] if c["name"] == winner), None)
    result = {"schema_version": STUDY_RESULT_SCHEMA_VERSION, "study": study, "calibration": rates,
              "runs": {n: {"run": r["run"], "returncode": r["returncode"], "seconds": r["seconds"], "ledger_validated": _ledger_ok(r),
                           "tokens_per_second": calibration.window_of(r.get("evidence")).get("tokens_per_second"),
                           "output_tail": r.get("output_tail", "")} for n, r in runs.items()},
              "ranking": ranking["ranking"], "chosen": winner,
              "chosen_overrides": list(chosen["overrides"]) if chosen else None,
              "prediction_error": _prediction_error(study, good)}
    with open(os.path.join(out_dir, "topology-study.json"), "w") as f:
        json.dump(result, f, indent=2, default=str)
    say(f"[topology] chosen {winner}; study written to {os.path.join(out_dir, 'topology-study.json')}")
    return result


def _prediction_error(study: dict, good: dict) -> dict:
    """Measured / predicted per split that ran: how far the balance rule is from the pipeline's real behaviour."""
    out = {}
    for c in study["candidates"]:
        run = good.get(c["name"])
        measured = calibration.window_of(run.get("evidence")).get("tokens_per_second") if run else None
        if measured and c.get("predicted_tokens_per_s"):
            out[c["name"]] = measured / c["predicted_tokens_per_s"]
    return out
