"""Shared-Target run with one failing experiment: the failure is fenced, the siblings finish.

    python tools/validation/multi_draft_faults.py --config MULTI_DRAFT_RECIPE.yaml --victim NAME --out DIR
           [--action raise|exit] [--step 1] [section.key=value ...]

The named experiment's trainer 0 raises (or its process exits) inside update ``--step``.  Expected: that experiment is
reported as failed and fenced (its readers never lease a slot again, rows that only waited for it go on to the others),
every other experiment completes all of its updates with a validated ledger, and all of them still trained on the same
rows.  Host-side injection only.  Prints one JSON verdict; exit code 0 when all of that holds.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from aspec_b200.config.train_config import load_config  # noqa: E402
from aspec_b200.multi_draft import compile_multi_draft_plan, run_multi_draft  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--victim", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--action", choices=("raise", "exit"), default="raise")
    ap.add_argument("--step", type=int, default=1)
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    plan = compile_multi_draft_plan(load_config(a.config, [*a.overrides, f"output_dir={a.out}"]))
    if a.victim not in plan.plans:
        ap.error(f"--victim must be one of {plan.names}")
    plan.plans[a.victim].runtime_args["fault_injection"] = {"kind": a.action, "step": a.step, "rank": 0}
    out = run_multi_draft(plan, log=lambda m: None)
    others = [n for n in plan.names if n != a.victim]
    steps = {n: out[n].get("completed_steps") for n in others}
    ledgers = [out[n].get("ledger", {}) for n in others]
    checks = {"victim_failed": "failed" in out[a.victim],
              "victim_fenced": a.victim in out["shared_source"]["fenced"],
              "siblings_completed": all(s and "failed" not in out[n] for n, s in steps.items()),
              "sibling_ledgers_validated": all(l.get("validated") for l in ledgers),
              "siblings_trained_the_same_rows": all(l.get("committed_work_ids") == ledgers[0].get("committed_work_ids") for l in ledgers)}
    print(json.dumps({"probe": "multi_draft_faults", "victim": a.victim, "action": a.action, "failure": out[a.victim].get("failed"),
                      "sibling_steps": steps, "checks": checks, "ok": all(checks.values())}))
    return 0 if all(checks.values()) else 1


if __name__ == "__main__":
    sys.exit(main())
