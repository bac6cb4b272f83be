"""Exact-resume probe: a run interrupted at update K and resumed must end in the same state as the uninterrupted run.

    python tools/validation/resume_replay.py --config RECIPE.yaml --steps 6 --at 3 --out DIR [section.key=value ...]

Three bounded runs of the ordinary train entry: ``whole`` (0 -> N, checkpoints at K and N), ``resumed`` (loads
``whole``'s checkpoint K, continues to N).  The two final checkpoints are compared section by section with the
checkpoint audit: weights, fp32 masters, both moments, the applied-step count, the scheduler, every rank's RNG streams and
the committed-work state.  Prints one JSON verdict; exit code 0 when every section agrees.

Bit-exactness of the Draft state presupposes bit-identical features.  Synthetic and stored features are; the in-framework
Target's features can differ in the last bit when rows are batched differently into one prefill (the reduction order of a
GEMM depends on its row count), and a resumed run batches its first rows differently from the uninterrupted run.  Pass
``inference.inference_batch_size=1 inference.inference_batch_tokens=0`` (one row per prefill) to check exact resume with
the live Target.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from aspec_b200 import train_entry  # noqa: E402
from aspec_b200.training.checkpoint_audit import checkpoint_hashes, compare  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--at", type=int, default=3)
    ap.add_argument("--out", required=True)
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    if not 0 < a.at < a.steps:
        ap.error("--at must lie strictly inside the run")
    common = [f"training.num_train_steps={a.steps}", "training.save_final_checkpoint=true", "dataset.eval_interval=0", *a.overrides]
    whole, resumed = os.path.join(a.out, "whole"), os.path.join(a.out, "resumed")
    train_entry.main(["--config", a.config, *common, f"training.save_interval={a.at}", f"output_dir={whole}"])
    first = os.path.join(whole, "checkpoints", f"iter_{a.at:07d}")
    train_entry.main(["--config", a.config, *common, "training.save_interval=0", f"training.load_path={first}",
                      f"output_dir={resumed}"])
    last = f"iter_{a.steps:07d}"
    diff = compare(checkpoint_hashes(os.path.join(whole, "checkpoints", last)),
                   checkpoint_hashes(os.path.join(resumed, "checkpoints", last)))
    print(json.dumps({"probe": "resume_replay", "steps": a.steps, "resumed_at": a.at, "exact": not diff,
                      "differing_sections": sorted(diff)}, default=str))
    return 0 if not diff else 1


if __name__ == "__main__":
    sys.exit(main())
