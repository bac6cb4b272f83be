"""Shared-Target run with one misbehaving experiment: the trouble stays with it, the siblings finish.

    python tools/validation/multi_draft_faults.py --config MULTI_DRAFT_RECIPE.yaml --victim NAME --out DIR
           [--action raise|exit|slow|cancel|cancel_blocked|stall|producer_fail] [--step 1] [section.key=value ...]

Actions, all injected on the host:

* ``raise`` / ``exit`` - the victim's trainer 0 raises, or its process exits, inside update ``--step``: the experiment is
  reported as failed and fenced (its readers never lease a slot again, rows that only waited for it go on to the others).
* ``slow`` - the victim's trainer 0 sleeps for a few seconds inside update ``--step``: nobody is fenced, every experiment
  (the victim too) completes all of its updates on the same rows.
* ``cancel`` - the operator cancels the victim once it has logged update ``--step``: it is fenced as cancelled.
* ``cancel_blocked`` - the victim's trainer 0 stops consuming at update ``--step`` (it sleeps for an hour), so its ring
  fills and the shared stream is waiting for one of its slots when the cancel arrives: the wait is abandoned, the
  siblings go on.
* ``stall`` - like ``cancel_blocked`` but nobody cancels: after ``transport.acquire_timeout_seconds`` without a free slot
  the stalled experiment is fenced by the stream itself.
* ``producer_fail`` - the Target engine fails after a few rows: every experiment ends with that error and no process is
  left behind.

In every case but the last, each experiment other than the victim must complete all of its updates with a validated
ledger, and all of them must have trained on the same rows.  Prints one JSON verdict; exit code 0 when that holds.
(reference: tools/validation/multi_draft_faults.py:30-63)
"""
import argparse
import json
import os
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from aspec_b200.config.train_config import load_config  # noqa: E402
from aspec_b200.multi_draft import compile_multi_draft_plan, run_multi_draft  # noqa: E402

ACTIONS = ("raise", "exit", "slow", "cancel", "cancel_blocked", "stall", "producer_fail")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--victim", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--action", choices=ACTIONS, default="raise")
    ap.add_argument("--step", type=int, default=1)
    ap.add_argument("--force-cpu", action="store_true")
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    plan = compile_multi_draft_plan(load_config(a.config, [*a.overrides, f"output_dir={a.out}"]))
    if a.victim not in plan.plans:
        ap.error(f"--victim must be one of {plan.names}")
    if a.force_cpu:
        for p in plan.plans.values():
            p.runtime_args.update(force_cpu=True)
    victim = plan.plans[a.victim].runtime_args
    cancel = {a.victim: threading.Event()}
    seen = {"cancel_at": None}

    def log(m: dict) -> None:
        # the operator's view: cancel once the victim has finished update ``--step`` (``cancel``), or once a sibling has
        # moved past the update in which the victim stopped consuming (``cancel_blocked``)
        if a.action == "cancel" and m.get("experiment") == a.victim and m.get("train/step") == a.step:
            cancel[a.victim].set()
        if a.action == "cancel_blocked" and m.get("experiment") != a.victim and int(m.get("train/step", -1)) >= a.step \
                and seen["cancel_at"] is None:
            # the victim stopped consuming inside this update: a little later its ring is full and the stream waits on it
            seen["cancel_at"] = m.get("train/step")
            threading.Timer(3.0, cancel[a.victim].set).start()

    if a.action in ("raise", "exit"):
        victim["fault_injection"] = {"kind": a.action, "step": a.step, "rank": 0}
    elif a.action == "slow":
        victim["fault_injection"] = {"kind": "sleep", "step": a.step, "rank": 0, "seconds": 4.0}
    elif a.action in ("cancel_blocked", "stall"):
        victim["fault_injection"] = {"kind": "sleep", "step": a.step, "rank": 0, "seconds": 3600.0}
    elif a.action == "producer_fail":
        for p in plan.plans.values():
            p.runtime_args["producer_fail_after"] = 3
    import psutil
    before = {p.pid for p in psutil.Process().children(recursive=True)}
    out = run_multi_draft(plan, log=log, cancel=cancel)
    others = [n for n in plan.names if n != a.victim]
    if a.action == "producer_fail":
        children = [c.pid for c in psutil.Process().children(recursive=True) if c.pid not in before and c.is_running()
                    and c.status() != psutil.STATUS_ZOMBIE
                    and "multiprocessing.resource_tracker" not in " ".join(c.cmdline())]      # this process's own helper
        checks = {"every_experiment_failed": all("failed" in out[n] for n in plan.names),
                  "failure_names_the_producer": all("producer" in str(out[n].get("failed", "")).lower()
                                                    or "inference" in str(out[n].get("failed", "")).lower() for n in plan.names),
                  "no_process_left": not children}
        print(json.dumps({"probe": "multi_draft_faults", "action": a.action, "failures": {n: str(out[n].get("failed"))[:160] for n in plan.names},
                          "checks": checks, "ok": all(checks.values())}))
        return 0 if all(checks.values()) else 1
    finishers = plan.names if a.action == "slow" else others
    steps = {n: out[n].get("completed_steps") for n in finishers}
    wanted = {n: int(plan.plans[n].runtime_args.get("num_train_steps") or 0) for n in finishers}
    ledgers = [out[n].get("ledger", {}) for n in finishers]
    checks = {"siblings_completed": all(s and "failed" not in out[n] and (not wanted[n] or s == wanted[n]) for n, s in steps.items()),
              "sibling_ledgers_validated": all(l.get("validated") for l in ledgers),
              "siblings_trained_the_same_rows": all(l.get("committed_work_ids") == ledgers[0].get("committed_work_ids") for l in ledgers)}
    fenced = out["shared_source"]["fenced"]
    if a.action == "slow":
        checks["nobody_fenced"] = not fenced
    else:
        checks["victim_fenced"] = a.victim in fenced
        if a.action in ("raise", "exit"):
            checks["victim_failed"] = "failed" in out[a.victim]
        elif a.action == "stall":
            checks["fenced_as_stalled"] = "stalled" in str(fenced.get(a.victim, "")).lower()
        else:
            checks["fenced_as_cancelled"] = "cancel" in str(fenced.get(a.victim, "")).lower()
    print(json.dumps({"probe": "multi_draft_faults", "victim": a.victim, "action": a.action, "failure": out[a.victim].get("failed"),
                      "sibling_steps": steps, "fenced": fenced, "checks": checks, "ok": all(checks.values())}))
    return 0 if all(checks.values()) else 1


if __name__ == "__main__":
    sys.exit(main())
