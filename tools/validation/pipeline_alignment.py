"""What reaches the Draft is what the Target computed for exactly those tokens.

    python tools/validation/pipeline_alignment.py --config RECIPE.yaml --out DIR [--steps 2] [--atol 1e-4] [overrides ...]

Runs a few updates of the recipe with the in-framework Target and step dumps switched on, then checks every dumped
micro-batch against an independent computation: the Target is rebuilt from the run's plan (same architecture, seed or
weights), every document of the row is found in the dataset by its work identity and prefilled ALONE, and the row the
trainer saw must hold, document by document in packing order, the document's own tokens, its own supervision mask and
the features of the Draft's captured layers at every position (and the post-norm last hidden state).  A shifted
offset, a swapped layer column, a stale ring slot or a mask from another document all show up as a mismatch.
An ``--out`` that already holds a run's dumps is checked again without running.  Prints one JSON verdict; exit code 1 on
any mismatch.
"""
import argparse
import glob
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from aspec_b200 import train_entry  # noqa: E402
from aspec_b200.config.train_config import config_to_flat_args, load_config  # noqa: E402
from aspec_b200.controller.training_controller import TrainingController  # noqa: E402
from aspec_b200.data.utils import unpack_loss_mask  # noqa: E402
from aspec_b200.inference.factory import target_config_from_args  # noqa: E402
from aspec_b200.models.target.dense import DenseTarget, TargetConfig  # noqa: E402
from aspec_b200.planning import compile_execution_plan  # noqa: E402
from aspec_b200.work_lifecycle import build_work_identity  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--atol", type=float, default=1e-4)
    ap.add_argument("--reference-seed", type=int, default=None,
                    help="build the independent Target from this seed instead of the run's (a self-test: it must then disagree)")
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    run = os.path.join(a.out, "run")
    overrides = [*a.overrides, "inference.inference_engine_type=native", f"training.num_train_steps={a.steps}",
                 "training.save_interval=0", "training.save_final_checkpoint=false", "dataset.eval_interval=0",
                 f"debug.save_debug_train_data={run}", f"debug.max_dump_steps={a.steps}", f"output_dir={run}"]
    if not glob.glob(os.path.join(run, "dumps", "step-*-rank*.pt")) and train_entry.main(["--config", a.config, *overrides]) != 0:
        print(json.dumps({"probe": "pipeline_alignment", "ok": False, "problem": "the run itself failed"}))
        return 1
    plan = compile_execution_plan(load_config(a.config, overrides))
    flat, draft = plan.to_runtime_args(), plan.draft_config
    if int(flat.get("draft_context_parallel_size", 1) or 1) != 1:
        print(json.dumps({"probe": "pipeline_alignment", "ok": False, "problem": "rows are sharded over a context-parallel group: "
                          "run the probe with draft_context_parallel_size=1"}))
        return 1
    layer_ids = [int(l) for l in draft["target_layer_ids"]]
    target = DenseTarget(TargetConfig(**target_config_from_args(flat, draft)))
    if flat.get("target_weights_path"):
        target.load_state_dict(torch.load(flat["target_weights_path"], map_location="cpu"), strict=True)
    else:
        target.init_random(int(flat.get("seed", 0)) if a.reference_seed is None else a.reference_seed)
    target = target.float().eval()
    controller = TrainingController(dict(flat), dp_size=1, consumers_per_row=1, algorithm=flat["draft_algorithm"])
    controller.load_dataset(None)
    by_work = {}
    for s in controller.samples:
        for epoch in range(max(int(flat.get("num_epochs", 1)), 1) + 1):
            by_work[build_work_identity(split="train", epoch=epoch, source_id=s["data_id"])["work_id"]] = s
    dumps = sorted(glob.glob(os.path.join(run, "dumps", "step-*-rank*.pt")))
    problems, rows, docs, worst = [], 0, 0, 0.0
    for path in dumps:
        b = torch.load(path, weights_only=False)["batch"]
        ids, feats = b["input_ids"][0], b["hidden_states"][0].float()
        last = b["last_hidden_states"][0].float() if "last_hidden_states" in b else None
        mask = b["loss_mask"].reshape(-1).float()
        lengths = list(b.get("packed_document_lengths") or [ids.numel()])
        rows += 1
        off = 0
        for meta, n in zip(b["_work"], lengths):
            docs += 1
            name = f"{os.path.basename(path)} document at {off}"
            src = by_work.get(meta["work_id"])
            if src is None:
                problems.append(f"{name}: work {meta['work_id'][:18]} is not a document of the dataset")
                off += n
                continue
            want_ids = src["input_ids"].reshape(-1)
            if n != want_ids.numel() or not torch.equal(ids[off:off + n].cpu(), want_ids):
                problems.append(f"{name}: tokens are not those of {src['data_id']}")
                off += n
                continue
            want_mask = unpack_loss_mask(src["packed_loss_mask"], n)
            if not torch.equal(mask[off:off + n].cpu(), want_mask.float()):
                problems.append(f"{name}: supervision mask is not that of {src['data_id']}")
            ref = target.prefill(want_ids, [n], layer_ids)
            err = float((feats[off:off + n].cpu() - ref["hidden_states"]).abs().max())
            if last is not None:
                err = max(err, float((last[off:off + n].cpu() - ref["last_hidden_states"]).abs().max()))
            worst = max(worst, err)
            scale = float(ref["hidden_states"].abs().max()) or 1.0
            if err > a.atol * max(scale, 1.0):
                problems.append(f"{name}: features differ from the document's own prefill by {err:.3g} (scale {scale:.3g})")
            off += n
        if off != ids.numel():
            problems.append(f"{os.path.basename(path)}: document lengths {lengths} do not cover the row's {ids.numel()} tokens")
    if not dumps:
        problems.append("the run wrote no step dumps")
    print(json.dumps({"probe": "pipeline_alignment", "ok": not problems, "rows": rows, "documents": docs,
                      "layers": layer_ids, "max_abs_feature_error": worst, "problems": problems[:12]}))
    return 0 if not problems else 1


if __name__ == "__main__":
    sys.exit(main())
