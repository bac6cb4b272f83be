"""Two Drafts share one (synthetic) Target on CPU: identical row stream, per-reader layer subsets, independent
ledgers and checkpoints, and fencing of a failed experiment while its sibling finishes
(reference: tests/test_multi_draft.py, tests/test_shared_source.py)."""
import os

import pytest

from aspec_b200.config.train_config import load_config
from aspec_b200.multi_draft import compile_multi_draft_plan, run_multi_draft

HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DSPARK = os.path.join(HERE, "aspec_b200", "config", "drafts", "dspark_tiny.json")
DFLASH = os.path.join(HERE, "aspec_b200", "config", "drafts", "dflash_tiny.json")


def _plan(tmp_path, second_extra=""):
    recipe = tmp_path / "recipe.yaml"
    recipe.write_text(f"""
model:
  draft_model_config: {DSPARK}
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 48
  synthetic_min_length: 32
  synthetic_max_length: 96
inference:
  inference_engine_type: synthetic
training:
  training_num_gpus_per_node: 1
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 128
  num_train_steps: 3
  learning_rate: 1e-3
  dspark_block_size: 4
  dspark_num_anchors: 16
  dflash_block_size: 4
  dflash_num_anchors: 16
  save_interval: 0
  seed: 7
transport:
  destination_ring_slots: 3
experiments:
  - name: spark
  - name: flash
    model:
      draft_model_config: {DFLASH}
{second_extra}
output_dir: {tmp_path / 'run'}
""")
    plan = compile_multi_draft_plan(load_config(str(recipe)))
    for p in plan.plans.values():
        p.runtime_args.update(synthetic_vocab_size=500, force_cpu=True)
    return plan


@pytest.mark.timeout(600)
def test_two_experiments_share_one_target_stream(tmp_path):
    plan = _plan(tmp_path)
    assert plan.union["contract"]["aux_hidden_state_layers"] == sorted(set(plan.union["contract"]["aux_hidden_state_layers"]))
    assert [v["layer_columns"] for v in plan.union["views"]][1] != [v["layer_columns"] for v in plan.union["views"]][0]
    logs = []
    out = run_multi_draft(plan, log=logs.append)
    assert out["spark"]["completed_steps"] == 3 and out["flash"]["completed_steps"] == 3
    # one Target pass per row, not one per experiment
    assert out["shared_source"]["rows_shared"] == 3 * 2              # 3 updates x 2 micro-batches, shared by both
    assert out["spark"]["ledger"]["committed_work_ids"] == out["flash"]["ledger"]["committed_work_ids"]
    assert {l["experiment"] for l in logs} == {"spark", "flash"}
    for name in ("spark", "flash"):
        assert os.path.isdir(os.path.join(tmp_path, "run", "experiments", name, "checkpoints"))


@pytest.mark.timeout(600)
def test_failed_experiment_is_fenced_and_sibling_finishes(tmp_path):
    plan = _plan(tmp_path)
    plan.plans["flash"].runtime_args["fault_injection"] = {"kind": "raise", "step": 1, "rank": 0}
    out = run_multi_draft(plan, log=lambda m: None)
    assert "failed" in out["flash"]
    assert out["spark"]["completed_steps"] == 3
    assert "flash" in out["shared_source"]["fenced"]


def test_experiments_must_agree_on_the_row_stream(tmp_path):
    with pytest.raises(ValueError, match="must agree on max_seq_length"):
        _plan(tmp_path, second_extra="    training:\n      max_seq_length: 64\n")


@pytest.mark.timeout(600)
def test_multi_draft_from_the_command_line_writes_per_experiment_metrics(tmp_path, capsys):
    import json
    from aspec_b200 import train_entry
    _plan(tmp_path)                                   # writes recipe.yaml
    recipe = tmp_path / "recipe.yaml"
    assert train_entry.main(["--config", str(recipe), "dataset.synthetic_vocab_size=500"]) == 0
    capsys.readouterr()
    run = tmp_path / "run"
    summary = json.loads((run / "multi-draft-summary.json").read_text())
    assert summary["spark"]["completed_steps"] == 3 and summary["flash"]["completed_steps"] == 3
    assert json.loads((run / "multi-draft-plan.json").read_text())["experiments"] == ["spark", "flash"]
    for name in ("spark", "flash"):
        rows = [json.loads(line) for line in (run / "experiments" / name / "runs" / "metrics.jsonl").read_text().splitlines()]
        assert [r["step"] for r in rows] == [0, 1, 2] and all("experiment" not in r for r in rows)
        assert json.loads((run / "experiments" / name / "tracking.json").read_text())["active"] == ["jsonl"]
        # every experiment's directory is a run directory of its own: configuration, plan, evidence, and a valid report
        evidence = json.loads((run / "experiments" / name / "evidence.json").read_text())
        assert evidence["state"] == "completed" and evidence["training_summary"]["completed_steps"] == 3
        assert evidence["sections"]["dataset_admission"]["admitted"] > 0
        assert evidence["plan_id"] == json.loads((run / "experiments" / name / "plan.json").read_text())["plan_id"]
        assert (run / "experiments" / name / "config.yaml").exists()
        assert train_entry.main(["--report", str(run / "experiments" / name), "--report-format", "json"]) == 0
        assert json.loads(capsys.readouterr().out)["valid"]
    session = json.loads((run / "evidence.json").read_text())
    assert session["schema_version"] == "aspec.multi-draft-evidence/v1" and session["state"] == "completed"
    assert {n: e["state"] for n, e in session["experiments"].items()} == {"spark": "completed", "flash": "completed"}
    assert session["plan_id"] == json.loads((run / "multi-draft-plan.json").read_text())["plan_id"]
    assert session["shared_source"]["rows_shared"] == 6
    assert json.loads((run / "cluster-preflight.json").read_text())["required_gpus"] == 2        # one Draft GPU per experiment


@pytest.mark.timeout(600)
def test_three_families_share_packed_rows_with_sharded_drafts(tmp_path):
    """DSpark, EAGLE3 with a pruned draft vocabulary and a 2-layer sliding-window DFlash read one packed row stream; every
    Draft is FULL_SHARD over two ranks.  The algorithms measure a document's work differently, so the rows are cut by
    the first experiment's measure; the pruned vocabulary comes from the admitted corpus."""
    import json
    eagle = tmp_path / "eagle.json"
    eagle.write_text(json.dumps(dict(
        architectures=["LlamaForCausalLMEagle3"], model_type="llama", hidden_size=64, intermediate_size=128, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, vocab_size=512, draft_vocab_size=128, num_hidden_layers=1, rope_theta=10000.0,
        max_position_embeddings=2048, target_hidden_size=64, target_num_hidden_layers=4, num_aux_hidden_states=3,
        target_layer_ids=[0, 1, 3])))
    flash = json.load(open(DFLASH))
    flash.update(num_hidden_layers=2, sliding_window=32)
    (tmp_path / "flash.json").write_text(json.dumps(flash))
    recipe = tmp_path / "recipe.yaml"
    recipe.write_text(f"""
model:
  draft_model_config: {DSPARK}
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 96
  synthetic_min_length: 32
  synthetic_max_length: 96
inference:
  inference_engine_type: synthetic
training:
  training_num_gpus_per_node: 2
  fsdp_strategy: FULL_SHARD
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 256
  dflash_packing: true
  num_train_steps: 2
  learning_rate: 1e-3
  dspark_block_size: 4
  dspark_num_anchors: 16
  dflash_block_size: 4
  dflash_num_anchors: 16
  ttt_length: 3
  save_interval: 0
  seed: 7
transport:
  destination_ring_slots: 5
experiments:
  - name: spark
  - name: eagle
    model:
      draft_model_config: {eagle}
  - name: flash
    model:
      draft_model_config: {tmp_path / 'flash.json'}
output_dir: {tmp_path / 'run'}
""")
    plan = compile_multi_draft_plan(load_config(str(recipe)))
    for p in plan.plans.values():
        p.runtime_args.update(synthetic_vocab_size=500, force_cpu=True)
    logs = []
    out = run_multi_draft(plan, log=logs.append)
    assert all(out[n].get("completed_steps") == 2 for n in ("spark", "eagle", "flash")), out
    # every Draft really trains: gradients reach the sharded optimizer of each family (the EAGLE3 Draft has no ``layers``
    # list and lives in the root unit whole)
    for n in ("spark", "eagle", "flash"):
        norms = [m["train/grad_norm"] for m in logs if m.get("experiment") == n and "train/grad_norm" in m]
        assert len(norms) == 2 and all(g > 0 for g in norms), (n, norms)
    assert out["shared_source"]["fenced"] == {} and out["shared_source"]["rows_shared"] == 2 * 2 * 2
    assert out["spark"]["ledger"]["committed_work_ids"] == out["eagle"]["ledger"]["committed_work_ids"]


@pytest.mark.timeout(600)
def test_a_reader_of_a_shared_stream_trains_like_the_same_draft_alone(tmp_path):
    """Same recipe once on its own and once as one of two experiments: identical loss and gradient-norm trajectory
    (shared rows, per-reader layer subsets of the union, row-keyed anchor draws)."""
    from aspec_b200.planning import compile_execution_plan
    from aspec_b200.train_entry import train_async_no_generation
    plan = _plan(tmp_path)
    for p in plan.plans.values():
        p.runtime_args.update(deterministic_anchor_sampling=True)
    logs = []
    run_multi_draft(plan, log=logs.append)
    shared = [(m["train/avg_loss"], m["train/grad_norm"]) for m in logs if m.get("experiment") == "spark" and "train/avg_loss" in m]
    alone_plan = plan.plans["spark"]
    flat = alone_plan.to_runtime_args()
    flat.update(output_dir=str(tmp_path / "alone"), deterministic_anchor_sampling=True)
    os.makedirs(flat["output_dir"], exist_ok=True)
    alone_logs = []
    train_async_no_generation(flat, alone_plan.draft_config, log=alone_logs.append)
    alone = [(m["train/avg_loss"], m["train/grad_norm"]) for m in alone_logs if "train/avg_loss" in m]
    assert len(shared) == len(alone) == 3
    for (a, b), (c, d) in zip(shared, alone):
        assert a == pytest.approx(c, rel=1e-6) and b == pytest.approx(d, rel=1e-6)


@pytest.mark.timeout(900)
def test_a_shared_target_run_resumes_every_experiment_from_its_own_checkpoint(tmp_path):
    """Four updates in one go against the last two of them again from every experiment's own checkpoint of update two:
    both experiments end with the same weights either way."""
    from aspec_b200.training.checkpoint_audit import checkpoint_hashes, compare

    def run(out, steps, extra=""):
        recipe = tmp_path / f"{os.path.basename(str(out))}.yaml"
        text = open(_recipe_text(tmp_path)).read().replace("num_train_steps: 3", f"num_train_steps: {steps}") \
            .replace("save_interval: 0", "save_interval: 2\n  deterministic_anchor_sampling: true" + extra)
        text = text[: text.index("output_dir:")] + f"output_dir: {out}\n"
        recipe.write_text(text)
        plan = compile_multi_draft_plan(load_config(str(recipe)))
        for p in plan.plans.values():
            p.runtime_args.update(synthetic_vocab_size=500, force_cpu=True)
        return run_multi_draft(plan, log=lambda m: None)

    whole = run(tmp_path / "whole", 4)
    middle = tmp_path / "whole" / "experiments" / "{experiment}" / "checkpoints" / "iter_0000002"
    second = run(tmp_path / "second", 4, f"\n  load_path: {middle}")
    assert whole["spark"]["completed_steps"] == 4
    assert second["spark"]["completed_steps"] == 2 and second["flash"]["completed_steps"] == 2
    # the root of an earlier run names every experiment's own directory (their latest checkpoints)
    from aspec_b200.multi_draft import experiment_load_path
    root = str(tmp_path / "whole")
    assert experiment_load_path({"load_path": root}, "flash") == os.path.join(root, "experiments", "flash")
    assert experiment_load_path({"load_path": str(middle)}, "spark").endswith("experiments/spark/checkpoints/iter_0000002")
    assert experiment_load_path({}, "spark") is None
    for name in ("spark", "flash"):
        a = checkpoint_hashes(str(tmp_path / "whole" / "experiments" / name / "checkpoints" / "iter_0000004"))
        b = checkpoint_hashes(str(tmp_path / "second" / "experiments" / name / "checkpoints" / "iter_0000004"))
        assert not compare(a, b), (name, sorted(compare(a, b)))


def _recipe_text(tmp_path):
    _plan(tmp_path)
    return str(tmp_path / "recipe.yaml")


@pytest.mark.timeout(600)
def test_experiments_evaluate_on_held_out_rows_that_the_target_produces_once(tmp_path):
    """Both experiments evaluate after updates 2 and 4: the first evaluation pulls the held-out rows through the shared
    stream (each row produced once for both readers), the second replays every experiment's own cache."""
    recipe_text = open(_recipe_text(tmp_path)).read().replace("num_train_steps: 3", "num_train_steps: 4") \
        .replace("  synthetic_max_length: 96", "  synthetic_max_length: 96\n  eval_data_path: synthetic\n  eval_interval: 2\n  eval_num_documents: 6")
    recipe = tmp_path / "eval.yaml"
    recipe.write_text(recipe_text)
    plan = compile_multi_draft_plan(load_config(str(recipe)))
    for p in plan.plans.values():
        p.runtime_args.update(synthetic_vocab_size=500, force_cpu=True)
    logs = []
    out = run_multi_draft(plan, log=logs.append)
    train_rows = 4 * 2                                           # updates x micro-batches, one trainer per experiment
    assert out["shared_source"]["rows_shared"] == train_rows + 6 and out["shared_source"]["fenced"] == {}
    for name in ("spark", "flash"):
        assert out[name]["completed_steps"] == 4 and out[name]["ledger"]["validated"]
        history = out[name]["evaluation"]["history"]
        assert [h["step"] for h in history] == [2, 4] and [h["from_cache"] for h in history] == [False, True]
        assert history[0]["metrics"]["eval/avg_loss"] == history[0]["metrics"]["eval/avg_loss"]          # a number
        assert out[name]["evaluation"]["best"]["step"] in (2, 4)
        assert os.path.isfile(os.path.join(plan.plans[name].runtime_args["output_dir"], "evaluation.json"))
        assert sum(1 for m in logs if m.get("experiment") == name and "eval/avg_loss" in m) == 2
    other = tmp_path / "other.yaml"
    other.write_text(recipe_text.replace("  - name: flash\n", "  - name: flash\n    dataset:\n      eval_interval: 3\n"))
    with pytest.raises(ValueError, match="must agree on eval_interval"):
        compile_multi_draft_plan(load_config(str(other)))


@pytest.mark.timeout(600)
def test_experiments_may_shard_the_shared_rows_over_different_context_parallel_degrees(tmp_path):
    """One experiment reads whole rows on one rank, the other shards every row over two context-parallel ranks: both
    have one data-parallel rank, so they plan the same rows; a different data-parallel width is refused."""
    cp2 = "    training:\n      training_num_gpus_per_node: 2\n      draft_context_parallel_size: 2"
    plan = _plan(tmp_path, second_extra=cp2)
    assert plan.consumer_offsets == {"spark": 0, "flash": 1}
    for p in plan.plans.values():
        p.runtime_args.update(deterministic_anchor_sampling=True, transport_destination_ring_slots=5)
    logs = []
    out = run_multi_draft(plan, log=logs.append)
    assert out["spark"]["completed_steps"] == out["flash"]["completed_steps"] == 3
    assert out["spark"]["ledger"]["committed_work_ids"] == out["flash"]["ledger"]["committed_work_ids"]
    assert out["shared_source"]["rows_shared"] == 3 * 2 and out["shared_source"]["fenced"] == {}
    assert all(m["train/grad_norm"] > 0 for m in logs if "train/grad_norm" in m)
    with pytest.raises(ValueError, match="same number of data-parallel ranks"):
        _plan(tmp_path, second_extra="    training:\n      training_num_gpus_per_node: 2")
