"""Train -> checkpoint -> exact resume -> export -> strict native load -> block proposal, on CPU."""
import json
import os

import pytest
import torch

from aspec_b200.commands.convert_to_hf import convert_checkpoint
from aspec_b200.config.draft_config import DSparkConfig
from aspec_b200.draft_artifact import BlockDraftConsumer, load_native_draft, validate_native_asset
from aspec_b200.models.draft.dspark import DSparkDraftModel
from aspec_b200.models.dspark import DSparkModel
from aspec_b200.training import checkpoint as ckpt
from aspec_b200.training.draft_trainer import DraftTrainer

ARGS = {"world_size": 1, "block_size": 4, "num_anchors": 8, "loss_decay_gamma": 4.0, "ce_loss_alpha": 0.1,
        "l1_loss_alpha": 0.9, "confidence_head_alpha": 1.0, "max_seq_length": 48, "micro_batch_size": 1,
        "draft_accumulation_steps": 2, "max_grad_norm": 1.0, "seed": 0, "anchor_sampling_scope": "row",
        "num_target_layers": 3}


def _build(seed=0):
    torch.manual_seed(seed)
    cfg = DSparkConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                       num_key_value_heads=2, vocab_size=128, num_target_layers=3, target_hidden_size=32,
                       target_num_hidden_layers=8, markov_rank=8, mask_token_id=127)
    draft = DSparkDraftModel(cfg)
    model = DSparkModel(draft, block_size=4, num_anchors=8, deterministic_anchor_sampling=True)
    head = torch.randn(128, 32) * 0.1
    trainer = DraftTrainer(model, head, lr=1e-2, total_steps=20, accumulation=2)
    return cfg, model, head, trainer


def _batch(i):
    g = torch.Generator().manual_seed(100 + i)
    T = 48
    return {"input_ids": torch.randint(0, 120, (1, T), generator=g), "loss_mask": torch.cat([torch.zeros(1, 12), torch.ones(1, 36)], 1),
            "hidden_states": torch.randn(1, T, 96, generator=g), "last_hidden_states": torch.randn(1, T, 32, generator=g)}


def test_train_resume_export_propose(tmp_path):
    out = str(tmp_path / "run")
    cfg, model, head, tr = _build()
    topo = ckpt.logical_training_topology(ARGS, cfg)
    losses = []
    for step in range(4):
        tr.train_update([_batch(2 * step), _batch(2 * step + 1)])
        losses.append(tr.metrics()["train/avg_loss"])
        if step == 1:
            ckpt.save(output_dir=out, step_id=2, model=model.draft_model, optimizer=tr.optimizer, draft_config=cfg,
                      topology=topo, global_step=tr.global_step)
            with pytest.raises((RuntimeError, FileNotFoundError)):
                ckpt.load(load_path=os.path.join(out, "checkpoints", ".iter_0000002.incomplete"), model=model.draft_model)
            ckpt.publish(output_dir=out, step_id=2, work_state={"committed_work_ids": ["a", "b"], "dataset_epoch": 0})
    assert all(l == l for l in losses)
    assert ckpt.latest_iteration(out) == 2
    it_dir = ckpt.resolve_checkpoint_dir(out)
    for name in ("model", "optimizer", "lr_scheduler", "rng", "meta.json", "draft_config.json", "work_state.json", "complete.json"):
        assert os.path.exists(os.path.join(it_dir, name))
    # exact resume in a fresh process-like state reproduces steps 2 and 3 bit for bit
    cfg2, model2, head2, tr2 = _build(seed=123)
    info = ckpt.load(load_path=out, model=model2.draft_model, optimizer=tr2.optimizer, topology=topo)
    assert info["next_step"] == 2 and info["work_state"]["committed_work_ids"] == ["a", "b"]
    tr2.global_step = info["global_step"]
    model2._step_counter = 4          # two micro-batches per update were consumed before the checkpoint
    tr2.lm_head_weight = head
    ckpt.finalize_load(info["checkpoint_dir"])
    resumed = []
    for step in range(2, 4):
        tr2.train_update([_batch(2 * step), _batch(2 * step + 1)])
        resumed.append(tr2.metrics()["train/avg_loss"])
    assert resumed == pytest.approx(losses[2:], rel=1e-6)
    # a different objective is refused, unless continual
    bad = ckpt.logical_training_topology({**ARGS, "block_size": 5}, cfg)
    with pytest.raises(ValueError):
        ckpt.load(load_path=out, model=model2.draft_model, optimizer=tr2.optimizer, topology=bad)
    ckpt.load(load_path=out, model=model2.draft_model, optimizer=tr2.optimizer, topology=bad, continual_training=True)
    # export both formats
    native = tmp_path / "native"
    man = convert_checkpoint(input_dir=tmp_path / "run", output_dir=native, artifact_format="aspec")
    assert man["schema_version"] == "aspec.serving-export/v1" and man["algorithm"] == "dspark"
    assert validate_native_asset(native)["model_sha256"] == man["model_sha256"]
    serving = tmp_path / "serving"
    convert_checkpoint(input_dir=tmp_path / "run", output_dir=serving, artifact_format="sglang")
    from safetensors.torch import load_file
    keys = set(load_file(str(serving / "model.safetensors")))
    assert "fc.weight" in keys and "hidden_norm.weight" in keys and "norm.weight" in keys
    with pytest.raises(FileExistsError):
        convert_checkpoint(input_dir=tmp_path / "run", output_dir=serving)
    # tamper -> refused
    loaded, _ = load_native_draft(native)
    consumer = BlockDraftConsumer(loaded, block_size=4)
    ids = torch.randint(0, 120, (1, 20))
    res = consumer.propose(ids, torch.randn(1, 20, 96), lm_head_weight=head)
    assert res["token_ids"].shape == (1, 4) and res["draft_confidence_logits"].shape == (1, 4)
    # hot reload: the same modules, new values; a proposal afterwards equals one from a freshly loaded consumer
    params_before = {n: p.data_ptr() for n, p in consumer.model.named_parameters()}
    with torch.no_grad():
        for p in consumer.model.parameters():
            p.add_(0.5)
    drifted = consumer.propose(ids, torch.randn(1, 20, 96, generator=torch.Generator().manual_seed(5)), lm_head_weight=head)
    consumer.update_weights_from_disk(native)
    assert {n: p.data_ptr() for n, p in consumer.model.named_parameters()} == params_before
    feats = torch.randn(1, 20, 96, generator=torch.Generator().manual_seed(5))
    fresh = BlockDraftConsumer(load_native_draft(native)[0], block_size=4).propose(ids, feats, lm_head_weight=head)
    again = consumer.propose(ids, feats, lm_head_weight=head)
    assert torch.equal(again["token_ids"], fresh["token_ids"])
    assert torch.allclose(again["draft_confidence_logits"], fresh["draft_confidence_logits"])
    del drifted
    cfgp = native / "config.json"
    cfgp.write_text(cfgp.read_text() + " ")
    with pytest.raises(ValueError):
        validate_native_asset(native)


def test_rotation_keeps_newest(tmp_path):
    root = tmp_path / "checkpoints"
    for i in (1, 2, 3, 4):
        (root / f"iter_{i:07d}").mkdir(parents=True)
    assert ckpt.rotate(str(tmp_path), keep_last=2, protect={1}) == [2]
    assert sorted(os.listdir(root)) == ["iter_0000001", "iter_0000003", "iter_0000004"]


def test_rng_file_is_bound_to_its_rank_and_world():
    import pytest
    from aspec_b200.training import checkpoint as C
    state = C._rng_state()
    assert state["rank"] == 0 and state["world_size"] == 1
    C._restore_rng(state)
    with pytest.raises(ValueError, match="offered to rank 0"):
        C._restore_rng(dict(state, rank=1, world_size=2))
    legacy = {k: v for k, v in state.items() if k not in ("rank", "world_size")}
    C._restore_rng(legacy)
