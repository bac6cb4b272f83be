"""Tensor-parallel Target on CPU (gloo ranks): a model sharded over two or four ranks is the unsharded model of the same
seed - same features, logits and cached decode passes - for dense and mixture-of-experts layers (the reference hands
``target_tp_size`` to its serving engine; here the in-framework Target shards itself)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aspec_b200.models.target.dense import DenseTarget, TargetConfig

DENSE = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=4, head_dim=16,
             vocab_size=200)
MOE = dict(DENSE, model_type="ling_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, num_shared_experts=1,
           first_k_dense_replace=1, n_group=2, topk_group=1)


def _inputs():
    g = torch.Generator().manual_seed(5)
    return torch.randint(0, 200, (13,), generator=g), [8, 5]


def _worker(rank, world, port, out, kw):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model = DenseTarget(TargetConfig(**kw), rank, world).init_random(1, std=0.2)
    ids, lengths = _inputs()
    full = model.prefill(ids, lengths, [0, 2], want_logits=True)
    cache = model.new_decode_cache(2, 16)
    a = model.extend(cache, [ids[:5], ids[8:10]], [0, 2])
    cache.accept(0, 5)
    cache.accept(1, 2)
    b = model.extend(cache, [ids[5:8], ids[10:]], [0, 2])
    torch.save({"logits": full["logits"], "features": full["hidden_states"], "last": full["last_hidden_states"],
                "cached": torch.cat([a["logits"][:5], b["logits"][:3], a["logits"][5:], b["logits"][3:]]),
                "agreed": model.agree(torch.tensor([rank + 7]))}, f"{out}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("kind,world", [("dense", 2), ("dense", 4), ("moe", 2)])
def test_a_sharded_target_is_the_whole_target(tmp_path, kind, world):
    kw = DENSE if kind == "dense" else MOE
    whole = DenseTarget(TargetConfig(**kw)).init_random(1, std=0.2)
    ids, lengths = _inputs()
    want = whole.prefill(ids, lengths, [0, 2], want_logits=True)
    out = str(tmp_path / "tp")
    mp.spawn(_worker, args=(world, 29300 + os.getpid() % 300, out, kw), nprocs=world, join=True)
    for rank in range(world):
        got = torch.load(f"{out}.{rank}")
        torch.testing.assert_close(got["logits"], want["logits"], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(got["features"], want["hidden_states"], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(got["last"], want["last_hidden_states"], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(got["cached"], want["logits"], rtol=1e-4, atol=1e-5)      # cached passes, this rank's heads only
        assert got["agreed"].item() == 7


def test_shards_of_a_checkpoint_are_the_seeded_shards_and_sizes_must_divide():
    whole = DenseTarget(TargetConfig(**MOE)).init_random(3, std=0.2)
    state = {**dict(whole.named_parameters()), **dict(whole.named_buffers())}
    for rank in range(2):
        part = DenseTarget(TargetConfig(**MOE), rank, 2)
        part.load_whole_state_dict(state)
        seeded = DenseTarget(TargetConfig(**MOE), rank, 2).init_random(3, std=0.2)
        for (name, p), (_, q) in zip(part.named_parameters(), seeded.named_parameters()):
            assert torch.equal(p, q), name
        assert part.memory_bytes() < 0.7 * whole.memory_bytes()
    with pytest.raises(ValueError, match="must divide num_key_value_heads"):
        DenseTarget(TargetConfig(**DENSE), 0, 8)


def test_the_planner_sizes_the_target_and_asks_for_tensor_parallelism_when_it_does_not_fit(tmp_path):
    import json
    from aspec_b200 import assets
    from aspec_b200.config.train_config import load_config
    from aspec_b200.planning import compile_execution_plan, estimate_target_memory
    small = json.load(open(assets.find_asset("targets/ling_moe_256e_12layer.json")))
    assert estimate_target_memory(small, 1, 32768)["fits"]
    big = dict(small, num_hidden_layers=32)
    assert not estimate_target_memory(big, 1, 32768)["fits"] and estimate_target_memory(big, 2, 32768)["fits"]
    assert estimate_target_memory(big, 2)["weights_bf16_per_gpu"] < 0.55 * estimate_target_memory(big, 1)["weights_bf16_per_gpu"]
    desc = tmp_path / "big.json"
    desc.write_text(json.dumps(big))
    recipe = assets.find_asset("ling_moe_256e_target_ep_draft.yaml")
    common = [f"model.target_model_config={desc}", f"output_dir={tmp_path / 'run'}"]
    with pytest.raises(ValueError, match="raise inference.target.tp_size"):
        compile_execution_plan(load_config(recipe, common))
    flat = load_config(recipe, common + ["inference.inference_num_gpus=4", "inference.target.tp_size=2",
                                         "training.training_num_gpus_per_node=4", "training.expert_parallel_size=4"])
    plan = compile_execution_plan(flat)
    assert any("tensor parallel over 2 GPUs" in c.reason for c in plan.capabilities)
    with pytest.raises(ValueError, match="must be a multiple of inference.target.tp_size"):
        compile_execution_plan(load_config(recipe, common + ["inference.inference_num_gpus=3", "inference.target.tp_size=2",
                                                             "training.training_num_gpus_per_node=4", "training.expert_parallel_size=4"]))
