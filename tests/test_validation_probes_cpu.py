"""The acceptance probes under tools/validation run end to end on CPU (reference: tools/validation/recipe_faults.py,
aspec/commands/_checkpoint_audit.py)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RECIPE = os.path.join(ROOT, "aspec_b200", "recipes", "quickstart_tiny.yaml")


def _probe(module, *args, expect=0):
    out = subprocess.run([sys.executable, "-m", f"tools.validation.{module}", *args], cwd=ROOT, capture_output=True, text=True,
                         timeout=560, env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert out.returncode == expect, out.stdout[-1500:] + out.stderr[-1500:]
    return json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])


@pytest.mark.timeout(600)
def test_resume_replay_is_exact_and_the_audit_sees_a_changed_state(tmp_path):
    res = _probe("resume_replay", "--config", RECIPE, "--steps", "4", "--at", "2", "--out", str(tmp_path / "r"))
    assert res["exact"] and res["differing_sections"] == []
    from aspec_b200.training.checkpoint_audit import checkpoint_hashes, compare
    a = checkpoint_hashes(str(tmp_path / "r" / "whole" / "checkpoints" / "iter_0000004"))
    b = checkpoint_hashes(str(tmp_path / "r" / "whole" / "checkpoints" / "iter_0000002"))
    assert a["model"]["coordinates"] > 0 and a["rng.rank-00000"]["rank"] == 0
    diff = compare(a, b)
    assert {"model", "optimizer.master", "optimizer.step", "lr_scheduler", "work_state"} <= set(diff)
    assert not compare(a, b, ignore=("model", "optimizer", "lr_scheduler", "work_state", "rng", "meta"))


@pytest.mark.timeout(600)
@pytest.mark.parametrize("action", ["trainer_raise", "producer_fail", "trainer_exit"])
def test_injected_host_faults_fail_the_run_and_leave_nothing_behind(tmp_path, action):
    res = _probe("recipe_faults", "--config", RECIPE, "--action", action, "--out", str(tmp_path / action))
    assert res["ok"], res


@pytest.mark.timeout(600)
def test_layouts_are_compared_update_by_update(tmp_path):
    # (the three sharding strategies are compared update by update in tests/test_pipeline_cpu.py)
    # context parallel 1 against 2: with row-derived anchor draws both layouts train on the same blocks
    res = _probe("layout_compare", "--config", RECIPE, "--out", str(tmp_path / "cp"), "--steps", "3", "--rtol", "1e-4",
                 "--a", "training.draft_context_parallel_size=1", "training.training_num_gpus_per_node=1",
                 "--b", "training.draft_context_parallel_size=2", "training.training_num_gpus_per_node=2", "--",
                 "transport.destination_ring_slots=5", "training.deterministic_anchor_sampling=true")
    assert res["metrics_agree"] and res["worst_relative_difference"] < 1e-5 and res["updates"] == [3, 3]
    # one rank accumulating four rows against two ranks accumulating two: the same documents per update, pooled the same way
    res = _probe("layout_compare", "--config", RECIPE, "--out", str(tmp_path / "dp"), "--steps", "3", "--rtol", "1e-4",
                 "--a", "training.training_num_gpus_per_node=1", "training.draft_accumulation_steps=4",
                 "--b", "training.training_num_gpus_per_node=2", "training.draft_accumulation_steps=2", "--",
                 "transport.destination_ring_slots=6", "training.deterministic_anchor_sampling=true", "dataset.length_group_size=1")
    assert res["metrics_agree"] and res["worst_relative_difference"] < 1e-5


@pytest.mark.timeout(600)
@pytest.mark.parametrize("action", ["exit", "stall", "producer_fail"])
def test_a_failing_experiment_is_fenced_while_its_siblings_finish(tmp_path, action):
    """``exit``: a trainer process of one experiment disappears.  ``stall``: one experiment stops consuming and nobody
    cancels it - the stream itself takes it out once its ring has been full for the acquire timeout.  ``producer_fail``:
    the shared Target fails - every experiment ends with that error and no process is left."""
    import yaml
    recipe = tmp_path / "multi.yaml"
    drafts = os.path.join(ROOT, "aspec_b200", "config", "drafts")
    recipe.write_text(yaml.safe_dump({
        "model": {"draft_model_config": os.path.join(drafts, "dspark_tiny.json")},
        "dataset": {"train_data_path": "synthetic", "synthetic_num_documents": 48, "synthetic_min_length": 32,
                    "synthetic_max_length": 96, "synthetic_vocab_size": 500},
        "inference": {"inference_engine_type": "synthetic"},
        "training": {"training_num_gpus_per_node": 1, "micro_batch_size": 1, "draft_accumulation_steps": 2, "max_seq_length": 128,
                     "num_train_steps": 3, "learning_rate": 1e-3, "dspark_block_size": 4, "dspark_num_anchors": 16,
                     "dflash_block_size": 4, "dflash_num_anchors": 16, "save_interval": 0, "seed": 7},
        "transport": {"destination_ring_slots": 3, "acquire_timeout_seconds": 5},
        "experiments": [{"name": "spark"}, {"name": "flash", "model": {"draft_model_config": os.path.join(drafts, "dflash_tiny.json")}},
                        {"name": "spark2"}],
    }))
    res = _probe("multi_draft_faults", "--config", str(recipe), "--victim", "flash", "--action", action, "--out", str(tmp_path / "run"),
                 "--force-cpu")
    assert res["ok"], res
    if action != "producer_fail":
        assert res["sibling_steps"] == {"spark": 3, "spark2": 3}, res


@pytest.mark.timeout(600)
def test_rows_at_the_trainer_are_the_targets_own_features_of_those_documents(tmp_path):
    """Packed rows, two Target engines, two trainers: every dumped micro-batch holds its documents' tokens, masks and
    captured-layer features in packing order."""
    recipe = tmp_path / "align.yaml"
    recipe.write_text("""
model:
  draft_model_config: dspark_tiny.json
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 48
  synthetic_min_length: 16
  synthetic_max_length: 48
  synthetic_vocab_size: 500
inference:
  inference_engine_type: native
  inference_num_gpus: 2
  inference_batch_size: 3
training:
  training_num_gpus_per_node: 2
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 128
  dflash_packing: true
  learning_rate: 1e-3
  dspark_block_size: 4
  dspark_num_anchors: 16
  seed: 11
""")
    res = _probe("pipeline_alignment", "--config", str(recipe), "--out", str(tmp_path / "a"))
    assert res["ok"] and res["rows"] == 4 and res["documents"] > res["rows"] and res["max_abs_feature_error"] < 1e-4
    # a Target of another seed is not the one whose features the trainer saw
    res = _probe("pipeline_alignment", "--config", str(recipe), "--out", str(tmp_path / "a"), "--reference-seed", "12", expect=1)
    assert not res["ok"] and "features differ" in res["problems"][0]


@pytest.mark.timeout(600)
def test_a_shared_target_run_resumes_exactly(tmp_path):
    drafts = os.path.join(ROOT, "aspec_b200", "config", "drafts")
    recipe = tmp_path / "md.yaml"
    recipe.write_text(f"""
model:
  draft_model_config: {drafts}/dspark_tiny.json
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 48
  synthetic_min_length: 32
  synthetic_max_length: 96
  synthetic_vocab_size: 500
inference:
  inference_engine_type: synthetic
training:
  training_num_gpus_per_node: 1
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 128
  learning_rate: 1e-3
  dspark_block_size: 4
  dspark_num_anchors: 16
  dflash_block_size: 4
  dflash_num_anchors: 16
  seed: 7
transport:
  destination_ring_slots: 3
experiments:
  - name: spark
  - name: flash
    model:
      draft_model_config: {drafts}/dflash_tiny.json
""")
    res = _probe("multi_draft_resume", "--config", str(recipe), "--out", str(tmp_path / "r"), "--force-cpu")
    assert res["ok"] and all(v["exact"] for v in res["experiments"].values())
