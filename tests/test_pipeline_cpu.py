"""Whole pipeline on CPU: driver + synthetic engine + 2 gloo trainer processes, checkpoint, resume, faults."""
import json
import os

import pytest
import torch

from aspec_b200.config.train_config import Config, config_to_flat_args, load_config
from aspec_b200.planning import compile_execution_plan
from aspec_b200.train_entry import train_async_no_generation

DRAFT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "aspec_b200", "config", "drafts", "dspark_tiny.json")


def _plan(tmp_path, extra=()):
    recipe = tmp_path / "recipe.yaml"
    recipe.write_text(f"""
model:
  draft_model_config: {DRAFT}
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 64
  synthetic_min_length: 32
  synthetic_max_length: 96
inference:
  inference_engine_type: synthetic
training:
  training_num_gpus_per_node: 2
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 128
  num_train_steps: 3
  learning_rate: 1e-3
  dspark_block_size: 4
  dspark_num_anchors: 16
  save_interval: 2
  seed: 7
transport:
  destination_ring_slots: 3
output_dir: {tmp_path / 'run'}
""")
    cfg = load_config(str(recipe), list(extra))
    return compile_execution_plan(cfg)


@pytest.mark.timeout(600)
def test_two_trainers_train_checkpoint_and_resume(tmp_path):
    plan = _plan(tmp_path)
    assert plan.plan_id.startswith("sha256:") and plan.policy["dp_size"] == 2
    flat = plan.to_runtime_args()
    flat.update(synthetic_vocab_size=500, force_cpu=True)
    os.makedirs(flat["output_dir"], exist_ok=True)
    logs = []
    summary = train_async_no_generation(flat, plan.draft_config, log=logs.append)
    assert summary["completed_steps"] == 3 and len(logs) == 3
    assert all(l["train/avg_loss"] == l["train/avg_loss"] for l in logs)
    for l in logs:                                   # where the update's time went
        assert all(l[f"perf/{k}"] >= 0 for k in ("data_time", "forward_time", "backward_time", "optimizer_time", "step_time"))
        assert l["perf/compute_time"] == pytest.approx(l["perf/forward_time"] + l["perf/backward_time"]) and l["perf/compute_time"] > 0
        assert l["perf/compute_time"] + l["perf/optimizer_time"] <= l["perf/step_wall_time"] * 1.05
    led = summary["ledger"]
    assert led["validated"] and led["committed_steps"] == [0, 1, 2] and len(led["committed_work_ids"]) == 12
    ck = os.path.join(flat["output_dir"], "checkpoints")
    assert sorted(d for d in os.listdir(ck) if d.startswith("iter_")) == ["iter_0000002", "iter_0000003"]
    ws = json.load(open(os.path.join(ck, "iter_0000002", "work_state.json")))
    assert len(ws["committed_work_ids"]) == 8
    # resume from iter 2: runs exactly one more step, on work that was not committed before
    flat2 = dict(flat, load_path=os.path.join(ck, "iter_0000002"), output_dir=str(tmp_path / "run2"), save_interval=0,
                 save_final_checkpoint=False)
    logs2 = []
    summary2 = train_async_no_generation(flat2, plan.draft_config, log=logs2.append)
    assert summary2["completed_steps"] == 1 and logs2[0]["train/step"] == 2
    assert not (set(summary2["ledger"]["committed_work_ids"]) & set(ws["committed_work_ids"]))
    assert logs2[0]["train/avg_loss"] == pytest.approx(logs[2]["train/avg_loss"], rel=1e-5)


@pytest.mark.timeout(300)
def test_trainer_failure_and_producer_failure_surface(tmp_path):
    plan = _plan(tmp_path)
    flat = plan.to_runtime_args()
    flat.update(synthetic_vocab_size=500, force_cpu=True, save_interval=0, save_final_checkpoint=False)
    os.makedirs(flat["output_dir"], exist_ok=True)
    from aspec_b200.runtime.actor import ActorError
    with pytest.raises(ActorError, match="injected failure at step 1"):
        train_async_no_generation(dict(flat, fault_injection={"kind": "raise", "step": 1, "rank": 1}), plan.draft_config,
                                  log=lambda m: None)
    with pytest.raises(RuntimeError, match="injected producer failure"):
        train_async_no_generation(dict(flat, producer_fail_after=3), plan.draft_config, log=lambda m: None)


@pytest.mark.timeout(300)
def test_step_deadline_terminates_trainers(tmp_path):
    plan = _plan(tmp_path)
    flat = plan.to_runtime_args()
    flat.update(synthetic_vocab_size=500, force_cpu=True, save_interval=0, save_final_checkpoint=False,
                optimizer_step_timeout_seconds=3.0, fault_injection={"kind": "sleep", "step": 1, "rank": 0, "seconds": 120})
    os.makedirs(flat["output_dir"], exist_ok=True)
    from aspec_b200.controller.loop import TrainerStepTimeoutError
    with pytest.raises(TrainerStepTimeoutError):
        train_async_no_generation(flat, plan.draft_config, log=lambda m: None)


@pytest.mark.timeout(600)
def test_full_shard_matches_replicate(tmp_path):
    """Same recipe under REPLICATE, SHARD_OPTIMIZER (optimizer state sharded) and FULL_SHARD (parameters and gradients
    sharded per layer too): identical losses, and the fully sharded run's checkpoint resumes."""
    losses = {}
    for strategy in ("REPLICATE", "SHARD_OPTIMIZER", "FULL_SHARD"):
        plan = _plan(tmp_path / strategy if (tmp_path / strategy).mkdir() is None else tmp_path, [f"training.fsdp_strategy={strategy}"])
        flat = plan.to_runtime_args()
        flat.update(synthetic_vocab_size=500, force_cpu=True, save_interval=2, save_final_checkpoint=False)
        os.makedirs(flat["output_dir"], exist_ok=True)
        logs = []
        train_async_no_generation(flat, plan.draft_config, log=logs.append)
        losses[strategy] = [l["train/avg_loss"] for l in logs]
        if strategy == "FULL_SHARD":
            ck = os.path.join(flat["output_dir"], "checkpoints", "iter_0000002")
            logs2 = []
            train_async_no_generation(dict(flat, load_path=ck, output_dir=str(tmp_path / "resumed"), save_interval=0),
                                      plan.draft_config, log=logs2.append)
            assert logs2[0]["train/step"] == 2
            assert logs2[0]["train/avg_loss"] == pytest.approx(logs[2]["train/avg_loss"], rel=1e-5)
    assert losses["FULL_SHARD"] == pytest.approx(losses["REPLICATE"], rel=1e-5)
    assert losses["SHARD_OPTIMIZER"] == pytest.approx(losses["REPLICATE"], rel=1e-5)


@pytest.mark.timeout(600)
def test_context_parallel_trainers_share_rows(tmp_path):
    """Two trainers forming one context-parallel group: every row goes to both, each takes half of the context and
    half of the blocks, and the work ledger sees two consumers per row."""
    plan = _plan(tmp_path, ["training.draft_context_parallel_size=2", "training.dspark_num_anchors=16"])
    assert plan.policy["dp_size"] == 1 and plan.policy["context_parallel"] == 2
    flat = plan.to_runtime_args()
    flat.update(synthetic_vocab_size=500, force_cpu=True, save_interval=0, save_final_checkpoint=False)
    os.makedirs(flat["output_dir"], exist_ok=True)
    logs = []
    summary = train_async_no_generation(flat, plan.draft_config, log=logs.append)
    assert summary["completed_steps"] == 3
    assert all(l["train/avg_loss"] == l["train/avg_loss"] and l["train/avg_loss"] > 0 for l in logs)
    assert summary["ledger"]["validated"] and len(summary["ledger"]["committed_work_ids"]) == 6


@pytest.mark.timeout(600)
def test_held_out_evaluation_runs_and_replays_from_the_trainer_cache(tmp_path):
    plan = _plan(tmp_path, ["dataset.eval_data_path=synthetic", "dataset.eval_interval=1"])
    flat = plan.to_runtime_args()
    flat.update(synthetic_vocab_size=500, force_cpu=True, save_interval=0, save_final_checkpoint=False, eval_num_documents=8,
                eval_decode_anchors_per_doc=2)
    os.makedirs(flat["output_dir"], exist_ok=True)
    logs = []
    summary = train_async_no_generation(flat, plan.draft_config, log=logs.append)
    evals = summary["evaluation"]
    assert [e["step"] for e in evals] == [1, 2, 3] and all(e["eval/avg_loss"] > 0 for e in evals)
    # train-with-decode: proposals of the live weights on the cached rows, at every evaluation
    assert all(e["eval/decode_proposals"] > 0 and 1.0 <= e["eval/decode_tau"] <= 7.0 for e in evals)
    record = json.load(open(os.path.join(flat["output_dir"], "evaluation.json")))
    assert [h["from_cache"] for h in record["history"]] == [False, True, True]      # the Target served the eval split once
    assert record["best"]["metric"] == "eval/avg_loss"
    assert summary["completed_steps"] == 3 and summary["ledger"]["validated"]


@pytest.mark.timeout(900)
def test_sequence_parallel_eagle3_pipeline_on_two_gloo_ranks(tmp_path):
    """EAGLE3 with ``sp_ulysses_size: 2``: two CPU trainer ranks share every row and report the loss of a one-rank run."""
    draft = tmp_path / "eagle3_tiny.json"
    draft.write_text(json.dumps(dict(
        architectures=["LlamaForCausalLMEagle3"], model_type="llama", hidden_size=32, intermediate_size=64, num_attention_heads=4,
        num_key_value_heads=2, head_dim=8, vocab_size=512, draft_vocab_size=512, target_hidden_size=32, target_num_hidden_layers=4,
        num_aux_hidden_states=3, rope_theta=10000.0, max_position_embeddings=256)))
    losses = {}
    for name, gpus, extra in (("one", 1, ""), ("sp2", 2, "  sp_ulysses_size: 2")):
        recipe = tmp_path / f"{name}.yaml"
        recipe.write_text(f"""
model:
  draft_model_config: {draft}
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 16
  synthetic_min_length: 40
  synthetic_max_length: 90
  shuffle_dataset: false
inference:
  inference_engine_type: synthetic
training:
  training_num_gpus_per_node: {gpus}
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 128
  num_train_steps: 2
  learning_rate: 1e-3
  ttt_length: 3
  save_interval: 0
  save_final_checkpoint: false
  seed: 3
{extra}
transport:
  destination_ring_slots: 4
output_dir: {tmp_path / name}
""")
        plan = compile_execution_plan(load_config(str(recipe), []))
        flat = plan.to_runtime_args()
        flat.update(synthetic_vocab_size=500, force_cpu=True)
        os.makedirs(flat["output_dir"], exist_ok=True)
        logs = []
        summary = train_async_no_generation(flat, plan.draft_config, log=logs.append)
        assert summary["completed_steps"] == 2 and summary["ledger"]["validated"]
        losses[name] = [l["train/avg_loss"] for l in logs]
    assert losses["sp2"] == pytest.approx(losses["one"], rel=1e-3)


@pytest.mark.timeout(600)
def test_checkpoint_at_every_epoch_end(tmp_path):
    """Eight documents, four per update: an epoch is two updates.  With ``save_per_epoch`` and no interval the run keeps a
    checkpoint where each epoch closed, and the final one is not written twice."""
    plan = _plan(tmp_path, ["dataset.synthetic_num_documents=8", "training.num_train_steps=5", "training.num_epochs=3",
                            "training.save_interval=0", "training.save_per_epoch=true", "training.max_checkpoints=10"])
    flat = plan.to_runtime_args()
    flat.update(synthetic_vocab_size=500, force_cpu=True)
    os.makedirs(flat["output_dir"], exist_ok=True)
    summary = train_async_no_generation(flat, plan.draft_config, log=lambda m: None)
    assert summary["completed_steps"] == 5
    ck = os.path.join(flat["output_dir"], "checkpoints")
    assert sorted(d for d in os.listdir(ck) if d.startswith("iter_")) == ["iter_0000002", "iter_0000004", "iter_0000005"]


@pytest.mark.timeout(600)
def test_rows_dispatched_several_updates_ahead(tmp_path):
    """``dispatch_ahead_updates`` keeps the producers several updates ahead of the trainers; the plan sizes the rings for
    it, every update trains on rows that really arrived, and the ledger validates."""
    plan = _plan(tmp_path, ["training.dispatch_ahead_updates=3", "training.num_train_steps=5"])
    flat = plan.to_runtime_args()
    assert flat["transport_destination_ring_slots"] >= 3 * 2 + 1
    flat.update(synthetic_vocab_size=500, force_cpu=True, save_interval=0, save_final_checkpoint=False)
    os.makedirs(flat["output_dir"], exist_ok=True)
    summary = train_async_no_generation(flat, plan.draft_config, log=lambda m: None)
    assert summary["completed_steps"] == 5 and summary["ledger"]["validated"]
    assert len(summary["ledger"]["committed_work_ids"]) == 5 * 2 * 2


@pytest.mark.timeout(300)
def test_unpacked_rows_of_several_documents_fit_their_ring_slot(tmp_path):
    """``micro_batch_size`` whole documents per row, each up to ``max_seq_length``: the slot is sized for all of them."""
    plan = _plan(tmp_path, ("training.micro_batch_size=2", "training.max_seq_length=100", "dataset.synthetic_min_length=70",
                            "dataset.synthetic_max_length=100", "training.num_train_steps=2", "training.training_num_gpus_per_node=1"))
    flat = plan.to_runtime_args()
    flat.update(synthetic_vocab_size=500, force_cpu=True, save_interval=0, save_final_checkpoint=False)
    os.makedirs(flat["output_dir"], exist_ok=True)
    logs = []
    summary = train_async_no_generation(flat, plan.draft_config, log=logs.append)
    assert summary["completed_steps"] == 2 and summary["ledger"]["validated"]
    assert all(l["perf/input_tokens"] > 2 * 2 * 70 for l in logs)                # 2 micro-batches x 2 documents of >= 70 tokens
