"""``quickstart {tiny,qwen3-8b} --output DIR [--steps N] [--plan]``: a bounded functional run - train, resume, export -
from a bundled profile (reference: aspec/commands/quickstart.py:30-110).  ``tiny`` needs no GPU and no model files;
``qwen3-8b`` runs the 1-layer Qwen3-8B-shaped recipe on the visible GPUs with a shape-bound random-init Target unless
``--target`` names a local checkpoint directory."""
from __future__ import annotations

import argparse
import json
import sys

PROFILES = {"tiny": "quickstart_tiny", "qwen3-8b": "qwen3_8b_dspark_1layer"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 quickstart", description=__doc__)
    ap.add_argument("model", choices=sorted(PROFILES))
    ap.add_argument("--output", required=True, help="fresh run directory")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--target", help="local Target checkpoint directory")
    ap.add_argument("--plan", action="store_true", help="print the execution plan only; starts nothing")
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    from aspec_b200.commands.recipes import catalog, run_acceptance
    overrides = list(a.overrides)
    if a.target:
        overrides.append(f"model.target_model_path={a.target}")
    if a.plan:
        from aspec_b200.train_entry import main as train_main
        return train_main(["--config", catalog()[PROFILES[a.model]]["config"], "--dry-run", f"output_dir={a.output}", *overrides])
    res = run_acceptance(PROFILES[a.model], a.output, a.steps, overrides)
    print(json.dumps({"output": a.output, "profile": a.model, "status": res["status"],
                      "asset": next((s.get("asset") for s in res["stages"] if s.get("asset")), None),
                      "scope": "functional train/resume/native export; not a quality claim"}, indent=2))
    return 0 if res["status"] == "passed" else 1


if __name__ == "__main__":
    sys.exit(main())
