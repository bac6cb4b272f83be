"""Train with decode on CPU: documents give prompts, the in-framework Target writes the responses (alone at first, then
verifying blocks of the live Draft after a weight sync), and the Draft trains on what was written (reference:
aspec/inference/engine/sgl_engine_decode.py:39-424, aspec/train_entry.py:330-338)."""
import json
import os

import pytest
import torch

from aspec_b200.config.train_config import load_config
from aspec_b200.controller.training_controller import TrainingController, prompt_of
from aspec_b200.planning import compile_execution_plan

RECIPE = """
model:
  draft_model_config: dspark_tiny.json
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 24
  synthetic_min_length: 24
  synthetic_max_length: 48
  synthetic_vocab_size: 500
inference:
  inference_engine_type: native
  inference_num_gpus: 1
training:
  training_num_gpus_per_node: 1
  micro_batch_size: 2
  draft_accumulation_steps: 2
  max_seq_length: 64
  num_train_steps: 4
  learning_rate: 1e-3
  dspark_block_size: 4
  dspark_num_anchors: 8
  save_interval: 0
  save_final_checkpoint: false
  seed: 3
  train_with_decode: true
decode:
  max_new_tokens: 12
  min_new_tokens: 4
  temperature: 0.7
  top_k: 50
  weight_sync_enabled: true
  weight_sync_interval: 2
"""


def test_the_prompt_is_everything_before_the_last_supervised_span():
    doc = {"input_ids": torch.arange(20), "packed_loss_mask": "4,3,5,6,2"}        # spans [4,7) and [12,18) are supervised
    assert prompt_of(doc).tolist() == list(range(12))
    assert prompt_of({"input_ids": torch.arange(5), "packed_loss_mask": "5"}).tolist() == list(range(5))
    assert prompt_of({"input_ids": torch.arange(5), "packed_loss_mask": "0,5"}).numel() == 0


def test_the_controller_plans_prompts_with_room_for_their_responses():
    args = {"max_seq_length": 32, "train_with_decode": True, "decode_max_new_tokens": 10, "decode_min_new_tokens": 2,
            "dspark_block_size": 4, "seed": 5, "decode_temperature": 0.5, "shuffle_dataset": False}
    docs = [{"data_id": "a", "input_ids": torch.arange(20), "packed_loss_mask": "8,12"},      # prompt 8, room 10
            {"data_id": "b", "input_ids": torch.arange(31), "packed_loss_mask": "30,1"},      # prompt 30: room 2 < block
            {"data_id": "c", "input_ids": torch.arange(30), "packed_loss_mask": "26,4"},      # prompt 26, room 6
            {"data_id": "d", "input_ids": torch.arange(9), "packed_loss_mask": "0,9"}]        # nothing to condition on
    c = TrainingController(args, dp_size=1, consumers_per_row=1, algorithm="dspark")
    assert c.load_dataset(docs) == 2
    assert c.admission["rejected"] == {"no_prompt": 1, "no_room_for_a_response": 1}
    req = c.row_request([0, 1], (0, 1))
    assert req.document_lengths == (8, 26) and req.input_ids.numel() == 34
    assert req.decode["max_new_tokens"] == [10, 6] and req.decode["temperature"] == 0.5
    again = TrainingController(args, dp_size=1, consumers_per_row=1, algorithm="dspark")
    again.load_dataset(docs)
    assert again.row_request([1], (0, 1)).decode["seeds"] == [req.decode["seeds"][1]]      # a document's noise is its own
    assert [s["length"] for s in c.samples] == [18, 32]


def test_the_planner_states_and_checks_the_mode(tmp_path):
    path = tmp_path / "r.yaml"
    path.write_text(RECIPE + f"output_dir: {tmp_path / 'run'}\n")
    plan = compile_execution_plan(load_config(str(path)))
    assert any(c.subsystem == "scope" and "train_with_decode" in c.reason for c in plan.capabilities)
    with pytest.raises(ValueError, match="needs the in-framework Target"):
        compile_execution_plan(load_config(str(path), ["inference.inference_engine_type=synthetic"]))
    with pytest.raises(ValueError, match="block Drafts only"):
        compile_execution_plan(load_config(str(path), ["model.draft_model_config=eagle3_qwen3_8b.json"]))
    compile_execution_plan(load_config(str(path), ["model.draft_model_config=eagle3_qwen3_8b.json", "decode.weight_sync_enabled=false"]))


@pytest.mark.timeout(900)
def test_a_run_decodes_its_own_responses_syncs_weights_and_repeats_exactly(tmp_path, capsys):
    from aspec_b200 import train_entry
    path = tmp_path / "r.yaml"
    path.write_text(RECIPE)

    def run(name, *overrides):
        assert train_entry.main(["--config", str(path), *overrides, f"output_dir={tmp_path / name}"]) == 0
        capsys.readouterr()
        rows = [json.loads(l) for l in open(tmp_path / name / "runs" / "metrics.jsonl")]
        return [r for r in rows if "train/avg_loss" in r], json.load(open(tmp_path / name / "evidence.json"))

    steps, evidence = run("a")
    summary = evidence["training_summary"]
    assert evidence["state"] == "completed" and summary["completed_steps"] == 4 and summary["ledger"]["validated"]
    assert summary["decode_weight_syncs"] == 2
    engine = summary["engines"][0]["decode"]
    assert engine["draft_loads"] == 2 and engine["generated_tokens"] == sum(s["decode/generated_tokens"] for s in steps)
    for s in steps:
        # every row is prompt + response: 4 documents per update, each with 4..12 written tokens
        assert 16 <= s["decode/generated_tokens"] <= 48 < s["perf/input_tokens"]
        assert s["decode/tokens_per_target_pass"] >= 1.0
    # the Target decodes alone until the first sync and verifies Draft blocks afterwards
    assert "decode/accepted_draft_tokens_per_round" not in steps[0] and engine["verify_rounds"] > 0
    assert (tmp_path / "a" / "scratch_draft_model" / "export_manifest.json").exists()
    # the text a document gets depends on the document and the seed alone: a second run repeats the first, also when
    # its engine decodes the documents of a call one at a time
    again, ev_b = run("b", "decode.max_running_requests=1")
    assert ev_b["training_summary"]["engines"][0]["decode"]["waves"] == 16
    assert [s["train/avg_loss"] for s in again] == pytest.approx([s["train/avg_loss"] for s in steps], rel=1e-6)
    assert [s["perf/input_tokens"] for s in again] == [s["perf/input_tokens"] for s in steps]
    # a Target engine spread over two tensor-parallel ranks writes the same text and features
    sharded, ev = run("tp", "inference.inference_num_gpus=2", "inference.target.tp_size=2")
    assert [s["perf/input_tokens"] for s in sharded] == [s["perf/input_tokens"] for s in steps]
    assert [s["train/avg_loss"] for s in sharded] == pytest.approx([s["train/avg_loss"] for s in steps], rel=1e-4)
    assert len(ev["training_summary"]["engines"]) == 1 and ev["sections"]["actor_initialization"]["inference_engine_count"] == 2


@pytest.mark.timeout(900)
def test_a_decoding_run_resumes_exactly_whatever_draft_its_engines_hold(tmp_path):
    """Interrupted after update 2 and resumed: the engines of the resumed run start without a Draft while those of the
    uninterrupted run verify blocks of the synced one, yet both write the same text (noise keyed by seed and token
    number) and end in the same checkpoint, section by section.  One document per Target call, so that the live Target's
    products do not depend on what else shared the call."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = tmp_path / "r.yaml"
    path.write_text(RECIPE)
    out = subprocess.run([sys.executable, "-m", "tools.validation.resume_replay", "--config", str(path), "--steps", "4", "--at", "2",
                          "--out", str(tmp_path / "rr"), "inference.inference_batch_size=1", "training.micro_batch_size=1",
                          "training.draft_accumulation_steps=4"], cwd=root, capture_output=True, text=True, timeout=800,
                         env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-1500:]
    verdict = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert verdict["exact"] and verdict["differing_sections"] == []
