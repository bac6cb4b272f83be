"""Sparse attention over a sharded context, two gloo ranks against the unsharded statements: global top-k from
per-shard candidates, log-softmax over entries spread over ranks, and selected-key attention merged by log-sum-exp -
including a rank whose shard is empty (reference: aspec/models/ops/distributed_sparse.py:54-241)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

N, T, K, HQ, HKV, D = 7, 60, 9, 4, 2, 16


def _problem():
    g = torch.Generator().manual_seed(0)
    scores = torch.randn(N, T, generator=g)
    lo = torch.tensor([0, 0, 5, 10, 30, 50, 12])
    hi = torch.tensor([60, 25, 5, 45, 33, 60, 40])
    q = torch.randn(N, HQ, D, generator=g)
    k = torch.randn(T, HKV, D, generator=g)
    v = torch.randn(T, HKV, D, generator=g)
    logits = torch.randn(N, T, generator=g)
    mask = torch.rand(N, T, generator=g) > 0.4
    mask[3] = False
    return scores, lo, hi, q, k, v, logits, mask


def _worker(rank, world, port, out, bounds):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.parallel.distributed_sparse import (distributed_log_softmax, distributed_selected_attention,
                                                        distributed_topk)
    scores, lo, hi, q, k, v, logits, mask = _problem()
    s0, s1 = bounds[rank]
    sel = distributed_topk(scores[:, s0:s1].contiguous(), lo, hi, K, s0)
    q = q.clone().requires_grad_()
    kl, vl = k[s0:s1].clone().requires_grad_(), v[s0:s1].clone().requires_grad_()
    per = -(-N // world)
    o0, o1 = min(rank * per, N), min((rank + 1) * per, N)
    out_rows = distributed_selected_attention(q, kl, vl, sel, s0, o0, o1, D ** -0.5)
    g = torch.Generator().manual_seed(9)
    dout = torch.randn(N, HQ, D, generator=g)
    out_rows.backward(dout[o0:o1])
    lg = logits[:, s0:s1].clone().requires_grad_()
    logp, valid = distributed_log_softmax(lg, mask[:, s0:s1])
    w = torch.randn(N, T, generator=g)
    (logp * w[:, s0:s1]).sum().backward()
    torch.save({"sel": sel, "out": out_rows.detach(), "rows": (o0, o1), "dq": q.grad, "dk": kl.grad, "dv": vl.grad,
                "logp": logp.detach(), "valid": valid, "dlogits": lg.grad}, f"{out}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("bounds", [[(0, 28), (28, 60)], [(0, 60), (60, 60)]])      # second case: an empty shard
def test_two_shards_match_the_unsharded_statements(tmp_path, bounds):
    out = str(tmp_path / "ds")
    mp.spawn(_worker, args=(2, 29650 + os.getpid() % 200, out, bounds), nprocs=2, join=True)
    from aspec_b200.ops.sparse_attention import selected_attention_reference, topk_select_reference
    scores, lo, hi, q, k, v, logits, mask = _problem()
    want_sel = topk_select_reference(scores, lo, hi, K)
    got = [torch.load(f"{out}.{r}") for r in range(2)]
    for r in range(2):
        assert torch.equal(got[r]["sel"], want_sel), r
    qr, kr, vr = q.clone().requires_grad_(), k.clone().requires_grad_(), v.clone().requires_grad_()
    ref, _ = selected_attention_reference(qr, kr, vr, want_sel, D ** -0.5)
    dout = torch.randn(N, HQ, D, generator=torch.Generator().manual_seed(9))
    ref.backward(dout)
    for r in range(2):
        o0, o1 = got[r]["rows"]
        assert torch.allclose(got[r]["out"], ref[o0:o1].detach(), atol=1e-5)
        s0, s1 = bounds[r]
        assert torch.allclose(got[r]["dk"], kr.grad[s0:s1], atol=1e-5)
        assert torch.allclose(got[r]["dv"], vr.grad[s0:s1], atol=1e-5)
    # every rank holds the gathered queries; the gradient of a query is the sum of what each rank computed for it
    assert torch.allclose(got[0]["dq"] + got[1]["dq"], qr.grad, atol=1e-5)
    lr = logits.clone().requires_grad_()
    x = lr.masked_fill(~mask, float("-inf"))
    full = torch.where(mask, torch.log_softmax(torch.where(mask.any(-1, keepdim=True), x, torch.zeros_like(x)), -1), torch.zeros_like(x))
    w = torch.randn(N, T, generator=torch.Generator().manual_seed(9).manual_seed(9))
    g = torch.Generator().manual_seed(9)
    torch.randn(N, HQ, D, generator=g)
    w = torch.randn(N, T, generator=g)
    (full * w).sum().backward()
    for r in range(2):
        s0, s1 = bounds[r]
        assert torch.allclose(got[r]["logp"], full[:, s0:s1].detach(), atol=1e-5)
        assert torch.equal(got[r]["valid"], mask.any(-1))
        assert torch.allclose(got[r]["dlogits"], lr.grad[:, s0:s1], atol=1e-5)
