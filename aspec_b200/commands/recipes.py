"""``recipes``: the catalog of bundled recipes and the acceptance workflow
``plan -> train the first half -> resume for the second half -> report -> export`` that proves a recipe's
train / checkpoint / exact-resume / export path end to end (reference: aspec/commands/recipes.py:272-459)."""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys
import time
from typing import Dict, List, Optional

_RECIPES = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "recipes")


def catalog() -> Dict[str, dict]:
    import yaml
    out = {}
    for path in sorted(glob.glob(os.path.join(_RECIPES, "*.yaml"))):
        raw = yaml.safe_load(open(path)) or {}
        t, inf = raw.get("training", {}), raw.get("inference", {})
        out[os.path.splitext(os.path.basename(path))[0]] = {
            "config": path, "draft": raw.get("model", {}).get("draft_model_config"),
            "engine": inf.get("inference_engine_type", "native"),
            "draft_gpus": int(t.get("training_num_gpus_per_node", 1)) * int(t.get("training_num_nodes", 1)),
            "target_gpus": int(inf.get("inference_num_gpus", 0)) if inf.get("inference_engine_type", "native") == "native" else 0,
            "experiments": [e["name"] for e in raw.get("experiments", [])]}
    return out


def run_acceptance(name: str, output: str, steps: int, overrides: Optional[List[str]] = None, log=print) -> dict:
    if steps < 2 or steps % 2:
        raise ValueError("--steps must be a positive even number >= 2")
    from aspec_b200.commands.convert_to_hf import convert_checkpoint
    from aspec_b200.config.train_config import load_config
    from aspec_b200.planning import compile_execution_plan
    from aspec_b200.reporting import build_run_report
    from aspec_b200.train_entry import main as train_main
    entry = catalog()[name]
    output = os.path.abspath(output)
    if os.path.exists(output):
        raise ValueError("Use a fresh output directory; existing runs are never changed.")
    os.makedirs(output)
    overrides = list(overrides or [])
    result = {"recipe": name, "scope": "bounded training/resume/native export", "status": "running", "steps": steps,
              "catalog": entry, "stages": [], "additional_gates": ["held-out quality", "serving decode", "fault injection"]}
    half = steps // 2

    def stage(label, fn):
        t0 = time.time()
        log(label)
        out = fn()
        result["stages"].append({"stage": label, "seconds": round(time.time() - t0, 2), **(out or {})})

    try:
        common = [f"training.num_train_steps={steps}", f"training.save_interval={half}", "training.save_final_checkpoint=true"]
        s1, s2 = os.path.join(output, "stage-1"), os.path.join(output, "stage-2")
        stage("plan", lambda: {"plan_id": compile_execution_plan(load_config(entry["config"], overrides + common + [f"output_dir={s1}"])).plan_id})
        stage("train first half", lambda: {"rc": train_main(["--config", entry["config"], *overrides, *common,
                                                              f"training.num_train_steps={half}", f"output_dir={s1}"])})
        ck = os.path.join(s1, "checkpoints", f"iter_{half:07d}")
        stage("resume second half", lambda: {"rc": train_main(["--config", entry["config"], *overrides, *common,
                                                               f"training.load_path={ck}", f"output_dir={s2}"])})
        stage("report", lambda: {"valid": build_run_report(s2).get("valid", False)})
        final = os.path.join(s2, "checkpoints", f"iter_{steps:07d}")
        asset = os.path.join(s2, "asset")
        stage("export", lambda: {"asset": asset, "schema": convert_checkpoint(input_dir=final, output_dir=asset,
                                                                                artifact_format="aspec")["schema_version"]})
        result["status"] = "passed"
    except BaseException as exc:                                 # noqa: BLE001 - recorded, then re-raised
        result["status"] = "failed"
        result["error"] = f"{type(exc).__name__}: {exc}"
        raise
    finally:
        with open(os.path.join(output, "acceptance.json"), "w") as f:
            json.dump(result, f, indent=2, default=str)
    return result


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 recipes", description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list")
    show = sub.add_parser("show")
    show.add_argument("name")
    plan = sub.add_parser("plan")
    plan.add_argument("name")
    plan.add_argument("overrides", nargs="*")
    acc = sub.add_parser("acceptance")
    acc.add_argument("name")
    acc.add_argument("--output", required=True)
    acc.add_argument("--steps", type=int, default=4)
    acc.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    cat = catalog()
    if a.cmd == "list":
        for name, e in cat.items():
            print(f"{name:32s} draft={e['draft']} engine={e['engine']} gpus={e['target_gpus']}T+{e['draft_gpus']}D"
                  + (f" experiments={e['experiments']}" if e["experiments"] else ""))
        return 0
    if a.name not in cat:
        raise ValueError(f"unknown recipe {a.name!r}; known: {sorted(cat)}")
    if a.cmd == "show":
        print(open(cat[a.name]["config"]).read())
        return 0
    if a.cmd == "plan":
        from aspec_b200.train_entry import main as train_main
        return train_main(["--config", cat[a.name]["config"], "--dry-run", *a.overrides])
    res = run_acceptance(a.name, a.output, a.steps, a.overrides)
    print(json.dumps({k: v for k, v in res.items() if k != "catalog"}, indent=2, default=str))
    return 0 if res["status"] == "passed" else 1


if __name__ == "__main__":
    sys.exit(main())
