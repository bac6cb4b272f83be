"""Ring attention on two and three gloo ranks against unsharded interval attention: forward, log-sum-exp and all three
gradients, with local-only extra keys (a Draft block / TTT keys) and queries that see nothing on some shards."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

S, E, HQ, HKV, D = 10, 3, 4, 2, 8          # rows per shard, extra local rows, heads


def _problem(R):
    g = torch.Generator().manual_seed(R)
    T = R * S
    q = torch.randn(R, S, HQ, D, generator=g)                 # S queries per rank
    k = torch.randn(T, HKV, D, generator=g)
    v = torch.randn(T, HKV, D, generator=g)
    ke = torch.randn(R, E, HKV, D, generator=g)               # extra rows, local to each rank
    ve = torch.randn(R, E, HKV, D, generator=g)
    iv = []
    for r in range(R):
        pos = r * S + torch.arange(S)
        lo = torch.randint(0, T // 2, (S,), generator=g).clamp(max=pos)          # causal window starting anywhere before
        n_extra = torch.randint(0, E + 1, (S,), generator=g)
        iv.append(torch.stack([lo, pos + 1, torch.full((S,), S), S + n_extra], -1).to(torch.int32))
    iv[0][0] = torch.tensor([0, 0, S, S])                     # a query that sees nothing at all
    dout = torch.randn(R, S, HQ, D, generator=g)
    return q, k, v, ke, ve, iv, dout


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aspec_b200.parallel.ring_attention import ring_attention
    q, k, v, ke, ve, iv, dout = _problem(world)
    ql = q[rank].clone().requires_grad_()
    kl = torch.cat([k[rank * S:(rank + 1) * S], ke[rank]]).clone().requires_grad_()
    vl = torch.cat([v[rank * S:(rank + 1) * S], ve[rank]]).clone().requires_grad_()
    o, lse = ring_attention(ql, kl, vl, iv[rank], S, D ** -0.5)
    o.backward(dout[rank])
    torch.save({"o": o.detach(), "lse": lse, "dq": ql.grad, "dk": kl.grad, "dv": vl.grad}, f"{out}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 3])
def test_ring_matches_unsharded_attention(tmp_path, world):
    from aspec_b200.ops.attention import interval_attention_reference
    out = str(tmp_path / "ring")
    mp.spawn(_worker, args=(world, 29500 + os.getpid() % 100 + world, out), nprocs=world, join=True)
    q, k, v, ke, ve, iv, dout = _problem(world)
    T = world * S
    kr, vr = k.clone().requires_grad_(), v.clone().requires_grad_()
    ker, ver = ke.clone().requires_grad_(), ve.clone().requires_grad_()
    for rank in range(world):
        got = torch.load(f"{out}.{rank}")
        qr = q[rank].clone().requires_grad_()
        # unsharded key array: the whole sequence, then this rank's extra rows
        keys, vals = torch.cat([kr, ker[rank]]), torch.cat([vr, ver[rank]])
        table = iv[rank].clone()
        table[:, 2:] += T - S
        ref, ref_lse = interval_attention_reference(qr, keys, vals, table, D ** -0.5)
        ref.backward(dout[rank])
        assert torch.allclose(got["o"], ref.detach(), atol=1e-5)
        fin = torch.isfinite(ref_lse)
        assert torch.equal(fin, torch.isfinite(got["lse"])) and torch.allclose(got["lse"][fin], ref_lse[fin].detach(), atol=1e-5)
        assert torch.allclose(got["dq"], qr.grad, atol=1e-5)
    for rank in range(world):
        got = torch.load(f"{out}.{rank}")
        assert torch.allclose(got["dk"][:S], kr.grad[rank * S:(rank + 1) * S], atol=1e-5)
        assert torch.allclose(got["dv"][:S], vr.grad[rank * S:(rank + 1) * S], atol=1e-5)
        assert torch.allclose(got["dk"][S:], ker.grad[rank], atol=1e-5)
        assert torch.allclose(got["dv"][S:], ver.grad[rank], atol=1e-5)
