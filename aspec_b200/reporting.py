"""``aspec --report RUN_DIR``: check that plan and evidence belong together and summarise the run
(reference: aspec/reporting.py:93-379)."""
from __future__ import annotations

import json
import os


def build_run_report(run_dir: str) -> dict:
    problems = []

    def load(name):
        p = os.path.join(run_dir, name)
        if not os.path.isfile(p):
            problems.append(f"missing {name}")
            return {}
        return json.load(open(p))

    plan, ev = load("plan.json"), load("evidence.json")
    if plan and ev and plan.get("plan_id") != ev.get("plan_id"):
        problems.append("evidence.json was written for a different plan")
    summary = ev.get("training_summary", {})
    ledger = summary.get("ledger", {})
    if ev and ev.get("state") != "completed":
        problems.append(f"run state is {ev.get('state')!r}")
    if ledger and not ledger.get("validated", False):
        problems.append("work ledger is not validated (residency, incomplete work or non-contiguous steps)")
    # a GPU run that launched something else than the plan chose (a fallback) is reported, not hidden
    observed = ev.get("capabilities_observed") or {}
    if (ev.get("accelerators") or {}).get("cuda"):
        for decision in plan.get("capabilities") or []:
            ran = observed.get(decision.get("subsystem"))
            if isinstance(ran, dict) and ran and decision.get("choice") not in ran:
                problems.append(f"plan chose {decision['choice']} for {decision['subsystem']}, the run launched {sorted(ran)}")
    ckpt_root = os.path.join(run_dir, "checkpoints")
    tracker = os.path.join(ckpt_root, "latest_checkpointed_iteration.txt")
    latest = int(open(tracker).read()) if os.path.isfile(tracker) else None
    return {"run_dir": os.path.abspath(run_dir), "valid": not problems, "problems": problems,
            "plan_id": plan.get("plan_id"), "algorithm": plan.get("workload", {}).get("algorithm"),
            "policy": plan.get("policy"), "state": ev.get("state"), "completed_steps": summary.get("completed_steps"),
            "throughput_window": summary.get("window"), "committed_work": len(ledger.get("committed_work_ids", [])),
            "dropped_tail_samples": summary.get("dropped_tail_samples"), "latest_checkpoint": latest,
            "capabilities": plan.get("capabilities"), "capabilities_observed": observed or None,
            "capabilities_activated": ev.get("capabilities_activated") or None,
            "dataset_admission": (ev.get("sections") or {}).get("dataset_admission"),
            "actor_initialization": (ev.get("sections") or {}).get("actor_initialization"),
            "cluster_preflight_state": ((ev.get("sections") or {}).get("cluster_preflight") or {}).get("state"),
            "cleanup": (ev.get("sections") or {}).get("cleanup"),
            "accelerators": ev.get("accelerators")}


def render_report(report: dict) -> str:
    lines = [f"run        {report['run_dir']}", f"valid      {report['valid']}",
             f"plan       {report.get('plan_id')}", f"algorithm  {report.get('algorithm')}",
             f"state      {report.get('state')}", f"steps      {report.get('completed_steps')}",
             f"committed  {report.get('committed_work')} documents", f"checkpoint iter {report.get('latest_checkpoint')}"]
    w = report.get("throughput_window") or {}
    if w.get("valid"):
        lines.append(f"throughput {w['tokens_per_second']:.1f} input tokens/s over {w['steps']} steady updates")
    adm = report.get("dataset_admission") or {}
    if adm:
        lines.append(f"dataset    {adm.get('admitted')} of {adm.get('source_rows')} source rows admitted"
                     + (f", rejected {adm['rejected']}" if adm.get("rejected") else ""))
    for name, act in (report.get("capabilities_activated") or {}).items():
        lines.append(f"activated  {name}: {act.get('planned') or ''} ({act.get('rule')})")
    for p in report.get("problems", []):
        lines.append(f"PROBLEM    {p}")
    return "\n".join(lines)
