"""Vocabulary-parallel head semantics on CPU: two gloo ranks with half of the head each reproduce the unsharded loss
terms and, summed over ranks, the unsharded gradients."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aspec_b200.ops.vocab_head import head_loss_reference

R, Tt, D, V, RK = 24, 10, 16, 64, 8


def _inputs():
    g = torch.Generator().manual_seed(3)
    return dict(hidden=torch.randn(R, D, generator=g), W=torch.randn(V, D, generator=g) * 0.3, W2=torch.randn(V, RK, generator=g) * 0.3,
                prev=torch.randn(R, RK, generator=g), teacher=torch.randn(Tt, D, generator=g),
                t_index=torch.randint(0, Tt, (R,), generator=g), labels=torch.randint(0, V, (R,), generator=g),
                weight=torch.rand(R, generator=g))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.parallel.vocab_parallel import vocab_parallel_head_loss_reference
    x = _inputs()
    shard = V // world
    sl = slice(rank * shard, (rank + 1) * shard)
    h, p = x["hidden"].clone().requires_grad_(True), x["prev"].clone().requires_grad_(True)
    w2 = x["W2"][sl].clone().requires_grad_(True)
    num, ce, l1 = vocab_parallel_head_loss_reference(h, x["W"][sl], x["labels"], x["weight"], vocab_offset=rank * shard, prev_emb=p,
                                                     markov_w2_shard=w2, teacher_hidden=x["teacher"], t_index=x["t_index"], a_ce=0.1, a_l1=0.9)
    num.backward()
    total = num.detach().clone()
    dist.all_reduce(total)
    dh, dp = h.grad.clone(), p.grad.clone()
    dist.all_reduce(dh)
    dist.all_reduce(dp)
    torch.save({"num": total, "ce": ce, "l1": l1, "dh": dh, "dp": dp, "dw2": w2.grad}, f"{out}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_match_the_unsharded_head(tmp_path):
    out = str(tmp_path / "vp")
    mp.spawn(_worker, args=(2, 29100 + os.getpid() % 500, out), nprocs=2, join=True)
    x = _inputs()
    h, p, w2 = x["hidden"].clone().requires_grad_(True), x["prev"].clone().requires_grad_(True), x["W2"].clone().requires_grad_(True)
    num, ce, l1, _ = head_loss_reference(h, x["W"], x["labels"], x["weight"], prev_emb=p, markov_w2=w2, teacher_hidden=x["teacher"],
                                         t_index=x["t_index"], a_ce=0.1, a_l1=0.9)
    num.backward()
    for rank in range(2):
        got = torch.load(f"{out}.{rank}")
        assert torch.allclose(got["num"], num.detach(), rtol=1e-5)
        assert torch.allclose(got["ce"], ce, atol=1e-5) and torch.allclose(got["l1"], l1, atol=1e-5)
        assert torch.allclose(got["dh"], h.grad, atol=1e-5) and torch.allclose(got["dp"], p.grad, atol=1e-5)
        shard = V // 2
        assert torch.allclose(got["dw2"], w2.grad[rank * shard:(rank + 1) * shard], atol=1e-5)
