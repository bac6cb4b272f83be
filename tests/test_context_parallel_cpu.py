"""Context-parallel wiring on CPU: two gloo ranks, each with half of the context rows and half of the blocks, must
reproduce the single-rank loss terms and (summed over ranks) the single-rank gradients."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aspec_b200.config.draft_config import DSparkConfig
from aspec_b200.models.draft.dspark import DSparkDraftModel
from aspec_b200.models.dspark import DSparkModel
from aspec_b200.ops.anchors import sample_anchor_positions

CFG = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           vocab_size=256, num_target_layers=3, target_hidden_size=64, target_num_hidden_layers=8, markov_rank=16,
           mask_token_id=255, layer_types=["full_attention", "sliding_attention"], sliding_window=24)


def _inputs():
    g = torch.Generator().manual_seed(5)
    T = 96
    ids = torch.randint(0, 250, (1, T), generator=g)
    feats = torch.randn(1, T, 192, generator=g)
    last = torch.randn(1, T, 64, generator=g)
    mask = torch.ones(1, T)
    mask[:, :12] = 0
    head = torch.randn(256, 64, generator=g) * 0.1
    anchors, keep = sample_anchor_positions(T, mask, 12, 4, generator=torch.Generator().manual_seed(9))
    return ids, feats, mask, head, last, anchors, keep


def _model():
    torch.manual_seed(0)
    return DSparkModel(DSparkDraftModel(DSparkConfig(**CFG)), block_size=4, num_anchors=12)


def _run(model):
    ids, feats, mask, head, last, anchors, keep = _inputs()
    out = model(ids, feats, mask, head, last_hidden_states=last, injected_anchors=anchors, injected_keep_mask=keep)
    num, den = out[6]
    num.backward()
    grads = {n: p.grad.clone() for n, p in model.draft_model.named_parameters() if p.grad is not None}
    return num.detach(), den.detach(), grads


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.parallel.cp_runtime import ContextParallel, attach
    model = _model()
    attach(model, ContextParallel(num_layers=2, max_queries=24, heads=4, head_dim=16))
    num, den, grads = _run(model)
    stats = torch.stack([num, den])
    dist.all_reduce(stats)
    for g in grads.values():
        dist.all_reduce(g)
    if rank == 0:
        torch.save({"stats": stats, "grads": grads}, out)
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_cp2_matches_single_rank(tmp_path):
    out = str(tmp_path / "cp.pt")
    mp.spawn(_worker, args=(2, 29900 + os.getpid() % 500, out), nprocs=2, join=True)
    got = torch.load(out)
    num, den, grads = _run(_model())
    assert torch.allclose(got["stats"][1], den)
    assert torch.allclose(got["stats"][0], num, rtol=1e-4, atol=1e-5)
    assert set(got["grads"]) == set(grads)
    for name, g in grads.items():
        assert torch.allclose(got["grads"][name], g, rtol=2e-3, atol=2e-5), name


def test_ulysses_attention_module_without_an_exchange_is_plain_gqa_attention():
    """The sequence-parallel block's single-GPU path (its own test reference on GPUs) against an explicit softmax."""
    import torch
    from aspec_b200.models.target.dense import DenseTarget
    from aspec_b200.parallel.ulysses_attention import UlyssesSelfAttention
    torch.manual_seed(0)
    m = UlyssesSelfAttention(32, 4, 2, 8)
    x = torch.randn(12, 32)
    iv = DenseTarget.causal_intervals([7, 5], "cpu")
    y = m(x, iv)
    q = (x @ m.q_proj.T).view(12, 4, 8)
    k = (x @ m.k_proj.T).view(12, 2, 8).repeat_interleave(2, 1)
    v = (x @ m.v_proj.T).view(12, 2, 8).repeat_interleave(2, 1)
    doc = torch.tensor([0] * 7 + [1] * 5)
    mask = (doc[:, None] == doc[None, :]) & (torch.arange(12)[:, None] >= torch.arange(12)[None, :])
    s = torch.einsum("qhd,khd->hqk", q, k) * 8 ** -0.5
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    want = torch.einsum("hqk,khd->qhd", p, v).reshape(12, 32) @ m.o_proj.T
    assert torch.allclose(y, want, atol=1e-5)


def _sp_eagle_worker(rank, world, port, out):
    import os
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.config.draft_config import AutoDraftModelConfig
    from aspec_b200.parallel.ulysses import CollectiveUlyssesExchange
    from aspec_b200.training.factory import build_training_model
    raw = dict(architectures=["LlamaForCausalLMEagle3"], model_type="llama", hidden_size=32, intermediate_size=64,
               num_attention_heads=4, num_key_value_heads=2, head_dim=8, vocab_size=96, draft_vocab_size=96, target_hidden_size=32,
               num_aux_hidden_states=3, rope_theta=10000.0, max_position_embeddings=256)
    torch.manual_seed(0)
    model = build_training_model(AutoDraftModelConfig.from_dict(raw), dict(ttt_length=3, seed=0), "cpu", torch.float32)
    model.train()
    T = 45                                                   # odd: padded to the group size
    g = torch.Generator().manual_seed(5)
    batch = dict(input_ids=torch.randint(0, 90, (1, T), generator=g), hidden_states_list=torch.randn(1, T, 96, generator=g),
                 loss_mask=torch.cat([torch.zeros(1, 6), torch.ones(1, T - 6)], 1),
                 lm_head_weight=torch.randn(96, 32, generator=g) * 0.2, last_hidden_states=torch.randn(1, T, 32, generator=g),
                 ctx_doc_ids=torch.cat([torch.zeros(1, 20), torch.ones(1, T - 20)], 1).long())
    if world > 1:
        model.draft_model.ulysses = CollectiveUlyssesExchange(rank, world)
        model.sequence_parallel = (rank, world, None)
    res = model(**batch)
    res[6][0].backward()
    num, den = res[6][0].detach().clone(), res[6][1].detach().clone()
    grads = {n: (p.grad.clone() if p.grad is not None else torch.zeros_like(p)) for n, p in model.draft_model.named_parameters()
             if p.requires_grad}
    if world > 1:
        dist.all_reduce(num)
        dist.all_reduce(den)
        for v in grads.values():
            dist.all_reduce(v)
    torch.save({"loss": num / den, "counts": res[4], "grads": grads}, f"{out}.{world}.{rank}")
    dist.destroy_process_group()


def test_sequence_parallel_eagle3_over_gloo_matches_one_process(tmp_path):
    """EAGLE3 with its rows sharded over two ranks (collective statement of the Ulysses exchange) gives the loss, the
    per-depth counts and the summed gradients of one process."""
    import os
    import torch
    import torch.multiprocessing as mp
    out = str(tmp_path / "sp")
    base = 29900 + os.getpid() % 80
    mp.spawn(_sp_eagle_worker, args=(1, base, out), nprocs=1, join=True)
    mp.spawn(_sp_eagle_worker, args=(2, base + 1, out), nprocs=2, join=True)
    one = torch.load(f"{out}.1.0")
    for rank in range(2):
        two = torch.load(f"{out}.2.{rank}")
        assert torch.allclose(two["loss"], one["loss"], rtol=1e-4)
        assert torch.equal(two["counts"], one["counts"])
        for name, g in one["grads"].items():
            assert torch.allclose(two["grads"][name], g, rtol=2e-3, atol=2e-5), name


# ---- DSA sparse stage under context parallelism ------------------------------------------------------------------
DSA_CFG = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=256, num_target_layers=3, target_hidden_size=64, target_num_hidden_layers=8, markov_rank=16,
               mask_token_id=255, layer_types=["deepseek_sparse_attention"], dsa_token_budget=10, dsa_index_n_heads=4,
               dsa_index_head_dim=16, dsa_q_lora_rank=16, dsa_rope_dim=8, dsa_training_stage="sparse")


def _dsa_model():
    torch.manual_seed(0)
    return DSparkModel(DSparkDraftModel(DSparkConfig(**DSA_CFG)), block_size=4, num_anchors=12)


def _dsa_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.parallel.cp_runtime import ContextParallel, attach
    model = _dsa_model()
    attach(model, ContextParallel(num_layers=1, max_queries=24, heads=4, head_dim=16))
    ids, feats, mask, head, last, anchors, keep = _inputs()
    res = model(ids, feats, mask, head, last_hidden_states=last, injected_anchors=anchors, injected_keep_mask=keep)
    num, den = res[6]
    num.backward()
    grads = {n: (p.grad.clone() if p.grad is not None else torch.zeros_like(p)) for n, p in model.draft_model.named_parameters()}
    stats = torch.stack([num.detach(), den.detach(), res[5]["dsa_indexer_loss"][0], res[5]["ce_loss"][0],
                         res[5]["l1_loss"][0], res[5]["confidence_loss"][0]])
    dist.all_reduce(stats)
    for g in grads.values():
        dist.all_reduce(g)
    if rank == 0:
        torch.save({"stats": stats, "grads": grads}, out)
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_dsa_sparse_stage_cp2_matches_single_rank(tmp_path):
    """A budget that really prunes: the global top-k over two shards, the merged selected-key attention and the
    selected-set KL must reproduce the one-rank loss terms and gradients."""
    out = str(tmp_path / "dsa_cp.pt")
    mp.spawn(_dsa_worker, args=(2, 29400 + os.getpid() % 200, out), nprocs=2, join=True)
    got = torch.load(out)
    model = _dsa_model()
    ids, feats, mask, head, last, anchors, keep = _inputs()
    res = model(ids, feats, mask, head, last_hidden_states=last, injected_anchors=anchors, injected_keep_mask=keep)
    num, den = res[6]
    num.backward()
    assert torch.allclose(got["stats"][1], den.detach())
    assert torch.allclose(got["stats"][3], res[5]["ce_loss"][0], rtol=1e-4, atol=1e-5)
    assert torch.allclose(got["stats"][2], res[5]["dsa_indexer_loss"][0], rtol=1e-4, atol=1e-5)
    # L1 / confidence terms pass through exp() of merged partial outputs: a little looser than the CE term
    assert torch.allclose(got["stats"][4], res[5]["l1_loss"][0], rtol=1e-3)
    assert torch.allclose(got["stats"][0], num.detach(), rtol=1e-3, atol=1e-5)
    bad = {}
    for name, p in model.draft_model.named_parameters():
        want = p.grad if p.grad is not None else torch.zeros_like(p)
        err = float((got["grads"][name] - want).abs().max() / want.abs().max().clamp_min(1e-9))
        if not torch.allclose(got["grads"][name], want, rtol=2e-3, atol=2e-5):
            bad[name] = round(err, 4)
    assert not bad, str(bad)


def _usp_eagle_worker(rank, world, port, out, u, r):
    """Ulysses x ring: ``u`` adjacent ranks exchange heads, ``r`` such blocks form the ring."""
    import os
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.config.draft_config import AutoDraftModelConfig
    from aspec_b200.parallel.ulysses import CollectiveUlyssesExchange
    from aspec_b200.training.factory import build_training_model
    raw = dict(architectures=["LlamaForCausalLMEagle3"], model_type="llama", hidden_size=32, intermediate_size=64,
               num_attention_heads=4, num_key_value_heads=2, head_dim=8, vocab_size=96, draft_vocab_size=96, target_hidden_size=32,
               num_aux_hidden_states=3, rope_theta=10000.0, max_position_embeddings=256)
    torch.manual_seed(0)
    model = build_training_model(AutoDraftModelConfig.from_dict(raw), dict(ttt_length=3, seed=0), "cpu", torch.float32)
    model.train()
    T = 45
    g = torch.Generator().manual_seed(5)
    batch = dict(input_ids=torch.randint(0, 90, (1, T), generator=g), hidden_states_list=torch.randn(1, T, 96, generator=g),
                 loss_mask=torch.cat([torch.zeros(1, 6), torch.ones(1, T - 6)], 1),
                 lm_head_weight=torch.randn(96, 32, generator=g) * 0.2, last_hidden_states=torch.randn(1, T, 32, generator=g),
                 ctx_doc_ids=torch.cat([torch.zeros(1, 20), torch.ones(1, T - 20)], 1).long())
    u_groups = [dist.new_group([b * u + i for i in range(u)]) if u > 1 else None for b in range(r)]
    ring_groups = [dist.new_group([b * u + i for b in range(r)]) for i in range(u)]
    model.draft_model.ulysses = CollectiveUlyssesExchange(rank % u, u, u_groups[rank // u])
    model.draft_model.ring = (rank // u, r, ring_groups[rank % u])
    model.sequence_parallel = (rank, world, None)
    res = model(**batch)
    res[6][0].backward()
    num, den = res[6][0].detach().clone(), res[6][1].detach().clone()
    grads = {n: (p.grad.clone() if p.grad is not None else torch.zeros_like(p)) for n, p in model.draft_model.named_parameters()
             if p.requires_grad}
    dist.all_reduce(num)
    dist.all_reduce(den)
    for v in grads.values():
        dist.all_reduce(v)
    torch.save({"loss": num / den, "counts": res[4], "grads": grads}, f"{out}.usp.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("u,r", [(2, 2), (1, 2)])
def test_ulysses_times_ring_eagle3_matches_one_process(tmp_path, u, r):
    """EAGLE3 (TTT depth keys stay local, depth-0 keys go round the ring) on ``u x r`` gloo ranks against one process."""
    import os
    import torch
    import torch.multiprocessing as mp
    out = str(tmp_path / "usp")
    base = 29200 + os.getpid() % 80
    mp.spawn(_sp_eagle_worker, args=(1, base, out), nprocs=1, join=True)
    mp.spawn(_usp_eagle_worker, args=(u * r, base + 1, out, u, r), nprocs=u * r, join=True)
    one = torch.load(f"{out}.1.0")
    for rank in range(u * r):
        two = torch.load(f"{out}.usp.{rank}")
        assert torch.allclose(two["loss"], one["loss"], rtol=1e-4)
        assert torch.equal(two["counts"], one["counts"])
        for name, g in one["grads"].items():
            assert torch.allclose(two["grads"][name], g, rtol=2e-3, atol=2e-5), name
