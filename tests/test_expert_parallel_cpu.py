"""Expert-parallel dispatch / combine semantics on CPU: two gloo ranks, each owning half of the experts, against the
replicated bank (forward, input gradient, expert weight gradients)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aspec_b200.models.draft.moe import ExpertBank, route_and_run

E, D, I, N, K = 4, 32, 16, 40, 2


def _full_bank():
    torch.manual_seed(0)
    return ExpertBank(E, D, I)


def _inputs(rank):
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(N, D, generator=g)
    sel = torch.randint(0, E, (N, K), generator=g)
    w = torch.rand(N, K, generator=g)
    dy = torch.randn(N, D, generator=g)
    return x, sel, w, dy


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = _full_bank()
    bank = ExpertBank(E, D, I, ep_rank=rank, ep_size=world)
    loc = E // world
    bank.gate_up_proj.data.copy_(full.gate_up_proj.data[rank * loc:(rank + 1) * loc])
    bank.down_proj.data.copy_(full.down_proj.data[rank * loc:(rank + 1) * loc])
    x, sel, w, dy = _inputs(rank)
    x.requires_grad_(True)
    y = route_and_run(bank, x, sel, w, dist.group.WORLD)
    y.backward(dy)
    torch.save({"y": y.detach(), "dx": x.grad, "dgu": bank.gate_up_proj.grad, "ddn": bank.down_proj.grad}, f"{out}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_match_the_replicated_bank(tmp_path):
    out = str(tmp_path / "ep")
    try:
        mp.spawn(_worker, args=(2, 29300 + os.getpid() % 500, out), nprocs=2, join=True)
    except Exception as exc:                                     # noqa: BLE001
        if "all_to_all" in str(exc) or "alltoall" in str(exc).lower():
            pytest.skip("this gloo build has no all_to_all")
        raise
    full = _full_bank()
    dgu = torch.zeros_like(full.gate_up_proj)
    ddn = torch.zeros_like(full.down_proj)
    for rank in range(2):
        x, sel, w, dy = _inputs(rank)
        x.requires_grad_(True)
        full.zero_grad()
        y = route_and_run(full, x, sel, w)
        y.backward(dy)
        got = torch.load(f"{out}.{rank}")
        assert torch.allclose(got["y"], y.detach(), atol=1e-5)
        assert torch.allclose(got["dx"], x.grad, atol=1e-5)
        dgu += full.gate_up_proj.grad
        ddn += full.down_proj.grad
    loc = E // 2
    for rank in range(2):
        got = torch.load(f"{out}.{rank}")
        assert torch.allclose(got["dgu"], dgu[rank * loc:(rank + 1) * loc], atol=1e-5)
        assert torch.allclose(got["ddn"], ddn[rank * loc:(rank + 1) * loc], atol=1e-5)


# ---- a whole training update with expert parallelism, against replicated experts ------------------------------
_RAW = dict(architectures=["DSparkDraftModel"], markov_rank=8, head_dim=16, target_layer_ids=[1, 3, 5], rope_theta=10000.0,
            max_position_embeddings=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, vocab_size=256, num_target_layers=3, target_hidden_size=64, target_num_hidden_layers=8,
            mask_token_id=255, ffn_type="qwen3_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32)
_ARGS = dict(block_size=4, dspark_block_size=4, dspark_num_anchors=8, seed=0)


def _train_batch(rank):
    g = torch.Generator().manual_seed(100 + rank)
    T = 48
    mask = torch.ones(1, T)
    mask[:, :10] = 0
    from aspec_b200.ops.anchors import sample_anchor_positions
    anchors, keep = sample_anchor_positions(T, mask, 8, 4, generator=g)
    return dict(input_ids=torch.randint(0, 250, (1, T), generator=g), hidden_states=torch.randn(1, T, 192, generator=g),
                loss_mask=mask, last_hidden_states=torch.randn(1, T, 64, generator=g), injected_anchors=anchors,
                injected_keep_mask=keep)


def _build():
    from aspec_b200.config.draft_config import AutoDraftModelConfig
    from aspec_b200.training.factory import build_training_model
    torch.manual_seed(0)
    model = build_training_model(AutoDraftModelConfig.from_dict(_RAW), _ARGS, "cpu", torch.float32)
    head = torch.randn(256, 64, generator=torch.Generator().manual_seed(5)) * 0.1
    return model, head


def _ep_train_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.parallel.expert_wiring import apply_expert_parallel, build_groups
    from aspec_b200.training.draft_trainer import DraftTrainer
    model, head = _build()
    group, replicas = build_groups(rank, world, world)
    plan = apply_expert_parallel(model.draft_model, rank, world, group, replicas)
    trainer = DraftTrainer(model, head, lr=1e-2, max_grad_norm=1.0, total_steps=10, warmup_ratio=0.0, accumulation=1,
                           device=torch.device("cpu"))
    trainer.optimizer.set_expert_parallel(plan.group, plan.ep_rank, plan.ep_size)
    trainer.expert_replica_group = plan.replica_group
    trainer.train_update([_train_batch(rank)])
    metrics = trainer.metrics()
    state = model.draft_model.state_dict()                      # collective: gathers the whole expert banks
    opt_state = trainer.optimizer.state_dict()
    if rank == 0:
        torch.save({"model": state, "grad_norm": metrics["train/grad_norm"], "loss": metrics["train/avg_loss"],
                    "master": opt_state["master"]}, out)
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_training_update_with_two_expert_parallel_ranks_matches_replicated_experts(tmp_path):
    out = str(tmp_path / "ep_train.pt")
    try:
        mp.spawn(_ep_train_worker, args=(2, 29800 + os.getpid() % 150, out), nprocs=2, join=True)
    except Exception as exc:                                     # noqa: BLE001
        if "all_to_all" in str(exc) or "alltoall" in str(exc).lower():
            pytest.skip("this gloo build has no all_to_all")
        raise
    from aspec_b200.training.draft_trainer import DraftTrainer
    model, head = _build()
    trainer = DraftTrainer(model, head, lr=1e-2, max_grad_norm=1.0, total_steps=10, warmup_ratio=0.0, accumulation=2,
                           device=torch.device("cpu"))
    trainer.train_update([_train_batch(0), _train_batch(1)])      # the two ranks' documents in one replicated update
    want = trainer.metrics()
    got = torch.load(out)
    assert got["loss"] == pytest.approx(want["train/avg_loss"], rel=1e-4)
    assert got["grad_norm"] == pytest.approx(want["train/grad_norm"], rel=1e-3)
    ref = model.draft_model.state_dict()
    assert set(ref) == set(got["model"])
    for name, t in ref.items():
        assert got["model"][name].shape == t.shape, name          # whole banks in the state dict
        assert torch.allclose(got["model"][name], t, atol=2e-5), name
    for name, t in trainer.optimizer.state_dict()["master"].items():
        assert torch.allclose(got["master"][name], t, atol=2e-5), name
