"""A shared-Target run that stops and resumes ends where the uninterrupted run ends, experiment by experiment.

    python tools/validation/multi_draft_resume.py --config RECIPE.yaml --out DIR [--steps 4] [--at 2] [overrides ...]

Runs the recipe (``experiments[]``) for ``--steps`` updates with a checkpoint at ``--at``, then a second time from every
experiment's own checkpoint of update ``--at`` (``training.load_path`` with ``{experiment}`` in it), and compares the
final checkpoints of every experiment section by section with the checkpoint audit: weights, masters, moments, step
counts, schedulers, RNG streams and committed work.  Readers of one row stream must all stand at the same row after the
restore; the runner refuses to start otherwise.  Prints one JSON verdict; exit code 1 if any experiment differs.
(reference: tools/validation/multi_draft_resume.py)
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from aspec_b200.config.train_config import load_config  # noqa: E402
from aspec_b200.multi_draft import compile_multi_draft_plan, run_multi_draft  # noqa: E402
from aspec_b200.training.checkpoint_audit import checkpoint_hashes, compare  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--at", type=int, default=2)
    ap.add_argument("--force-cpu", action="store_true")
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    if not 0 < a.at < a.steps:
        ap.error("--at must lie strictly inside the run")
    whole, resumed = os.path.join(a.out, "whole"), os.path.join(a.out, "resumed")
    common = [*a.overrides, f"training.num_train_steps={a.steps}", "training.save_final_checkpoint=true", "dataset.eval_interval=0",
              "training.deterministic_anchor_sampling=true"]

    def run(extra):
        plan = compile_multi_draft_plan(load_config(a.config, [*common, *extra]))
        if a.force_cpu:
            for p in plan.plans.values():
                p.runtime_args.update(force_cpu=True)
        return plan, run_multi_draft(plan, log=lambda m: None)

    plan, first = run([f"training.save_interval={a.at}", f"output_dir={whole}"])
    middle = os.path.join(whole, "experiments", "{experiment}", "checkpoints", f"iter_{a.at:07d}")
    _, second = run(["training.save_interval=0", f"training.load_path={middle}", f"output_dir={resumed}"])
    last = f"iter_{a.steps:07d}"
    verdict = {}
    for name in plan.names:
        diff = compare(checkpoint_hashes(os.path.join(whole, "experiments", name, "checkpoints", last)),
                       checkpoint_hashes(os.path.join(resumed, "experiments", name, "checkpoints", last)))
        verdict[name] = {"exact": not diff, "differing_sections": sorted(diff),
                         "updates": [first[name].get("completed_steps"), second[name].get("completed_steps")]}
    ok = all(v["exact"] and v["updates"] == [a.steps, a.steps - a.at] for v in verdict.values())
    print(json.dumps({"probe": "multi_draft_resume", "ok": ok, "steps": a.steps, "resumed_at": a.at, "experiments": verdict}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
