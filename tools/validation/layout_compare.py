"""Two parallel / sharding / packing layouts of one recipe must train the same model.

    python tools/validation/layout_compare.py --config RECIPE.yaml --out DIR --steps 4
           --a training.fsdp_strategy=REPLICATE --b training.fsdp_strategy=FULL_SHARD [--rtol 1e-5] [common overrides ...]

Runs the recipe twice through the ordinary train entry (``--a`` overrides, then ``--b`` overrides) and compares the
logged loss and gradient-norm trajectories update by update, then the final checkpoints' weights and optimizer state with
the checkpoint audit when both layouts keep the same world size (bit-equal layouts) or within ``--rtol`` on the metrics
(layouts that change the order of floating-point sums).  Typical pairs: REPLICATE / SHARD_OPTIMIZER / FULL_SHARD;
``draft_context_parallel_size`` 1 / 2; ``dflash_packing`` on / off with one document per row.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from aspec_b200 import train_entry  # noqa: E402
from aspec_b200.training.checkpoint_audit import checkpoint_hashes, compare  # noqa: E402

KEYS = ("train/avg_loss", "train/grad_norm", "train/avg_acc")


def _trajectory(run_dir: str):
    rows = []
    with open(os.path.join(run_dir, "runs", "metrics.jsonl")) as f:
        for line in f:
            rec = json.loads(line)
            if any(k in rec for k in KEYS):
                rows.append({k: rec.get(k) for k in KEYS})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--a", nargs="+", required=True)
    ap.add_argument("--b", nargs="+", required=True)
    ap.add_argument("--rtol", type=float, default=1e-5)
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    common = [f"training.num_train_steps={a.steps}", "training.save_interval=0", "training.save_final_checkpoint=true",
              "dataset.eval_interval=0", *a.overrides]
    runs = {}
    for tag, extra in (("a", a.a), ("b", a.b)):
        out = os.path.join(a.out, tag)
        train_entry.main(["--config", a.config, *common, *extra, f"output_dir={out}"])
        runs[tag] = out
    ta, tb = _trajectory(runs["a"]), _trajectory(runs["b"])
    worst = 0.0
    for ra, rb in zip(ta, tb):
        for k in KEYS:
            if ra.get(k) is not None and rb.get(k) is not None:
                worst = max(worst, abs(ra[k] - rb[k]) / max(abs(ra[k]), 1e-12))
    last = f"iter_{a.steps:07d}"
    ha = checkpoint_hashes(os.path.join(runs["a"], "checkpoints", last))
    hb = checkpoint_hashes(os.path.join(runs["b"], "checkpoints", last))
    diff = compare(ha, hb, ignore=("rng", "meta", "work_state"))
    ok = len(ta) == len(tb) == a.steps and worst <= a.rtol
    print(json.dumps({"probe": "layout_compare", "a": a.a, "b": a.b, "updates": [len(ta), len(tb)],
                      "worst_relative_difference": worst, "rtol": a.rtol, "metrics_agree": ok,
                      "state_sections_bit_equal": not diff, "differing_sections": sorted(diff)}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
