"""Vocabulary-parallel head: two ranks emulated on one GPU (phases interleaved, no kernel waits on another) must
reproduce the unsharded fused head and the fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_emulated_ranks_match_the_unsharded_head():
    from aspec_b200.ops.vocab_head import head_loss, head_loss_reference
    from aspec_b200.parallel.vocab_parallel import VocabParallelHead, VocabShardWorkspace
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    R, Tt, D, V, rk, world = 200, 96, 256, 4096, 32, 2
    bf = torch.bfloat16
    hidden = (torch.randn(R, D, device=dev) * 0.5).to(bf)
    W = (torch.randn(V, D, device=dev) * 0.05).to(bf)
    W2 = (torch.randn(V, rk, device=dev) * 0.05).to(bf)
    prev = (torch.randn(R, rk, device=dev) * 0.5).to(bf)
    teacher = (torch.randn(Tt, D, device=dev) * 0.5).to(bf)
    t_index = torch.randint(0, Tt, (R,), device=dev, dtype=torch.int32)
    labels = torch.randint(0, V, (R,), device=dev)
    weight = torch.rand(R, device=dev)
    weight[::7] = 0
    kw = dict(a_ce=0.1, a_l1=0.9)
    # unsharded fused head with gradients
    h1 = hidden.clone().requires_grad_(True)
    p1 = prev.clone().requires_grad_(True)
    w2_1 = W2.clone().requires_grad_(True)
    num1, ce1, l11, cor1 = head_loss(h1, W, labels, weight, prev_emb=p1, markov_w2=w2_1, teacher_hidden=teacher, t_index=t_index, **kw)
    num1.backward()
    # sharded, ranks interleaved phase by phase
    ws = [VocabShardWorkspace(256, 128, D, rk, world, device=dev) for _ in range(world)]
    heads = [VocabParallelHead(r, world, V, ws) for r in range(world)]
    shards = [(h.shard_rows(W).contiguous(), h.shard_rows(W2).contiguous()) for h in heads]
    for h, (w, w2) in zip(heads, shards):
        h.logits(hidden, w, prev, w2, teacher)
    for h in heads:
        h.statistics(labels, weight, t_index, kw["a_ce"], kw["a_l1"])
    outs = [h.gradient() for h in heads]
    for ce, l1, cor in outs:
        assert torch.allclose(ce, ce1, rtol=2e-3, atol=2e-3)
        assert torch.allclose(l1, l11, rtol=2e-3, atol=2e-3)
        assert (cor != cor1).float().mean() < 0.01
    ref = head_loss_reference(hidden, W, labels, weight, prev_emb=prev, markov_w2=W2, teacher_hidden=teacher, t_index=t_index, **kw)
    assert torch.allclose(outs[0][0], ref[1], rtol=3e-2, atol=3e-2)
    for h, (w, w2) in zip(heads, shards):
        h.scatter_partials(w, w2)
    for h in heads:
        dh, dprev = h.reduce_partials(rk)
        assert torch.allclose(dh.float(), h1.grad.float(), rtol=5e-2, atol=2e-3 * h1.grad.float().abs().max().item() + 1e-6)
        assert torch.allclose(dprev.float(), p1.grad.float(), rtol=5e-2, atol=2e-3 * p1.grad.float().abs().max().item() + 1e-6)


def test_scatter_epilogue_routes_column_blocks():
    from aspec_b200.ops import gemm as G
    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    a = (torch.randn(300, 256, device=dev) * 0.3).to(torch.bfloat16)
    b = (torch.randn(384, 256, device=dev) * 0.3).to(torch.bfloat16)
    dests = [torch.zeros(300, 128, device=dev, dtype=torch.bfloat16) for _ in range(3)]
    G.gemm(a, b, mirrors=dests, scatter_cols=128)
    ref = (a.float() @ b.float().T)
    for m, d in enumerate(dests):
        assert torch.allclose(d.float(), ref[:, m * 128:(m + 1) * 128], rtol=2e-2, atol=2e-2)
