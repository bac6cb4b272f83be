"""FULL_SHARD optimizer: the sharded protocol must produce the replicated optimizer's parameters.
CPU: two gloo ranks.  GPU: the two peer-memory kernels with two emulated ranks' buffers on one device."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aspec_b200.training.optimizer import BF16Optimizer
from aspec_b200.training.sharded_optimizer import ShardedBF16Optimizer, shard_bounds


def _model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(24, 40, bias=False), torch.nn.Linear(40, 13, bias=False))


def _grads(rank, step, model):
    g = torch.Generator().manual_seed(100 * step + rank)
    return [torch.randn(p.shape, generator=g) for p in model.parameters()]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model = _model()
    opt = ShardedBF16Optimizer(model, lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
    for step in range(3):
        for p, g in zip(model.parameters(), _grads(rank, step, model)):
            p.main_grad.add_(g)
        opt.set_grad_scale(0.5)
        norm = opt.step()
    if rank == 0:
        torch.save({"params": [p.detach().clone() for p in model.parameters()], "norm": norm,
                    "full": opt.full_state()["master"]}, out)
    else:
        opt.full_state()
    dist.destroy_process_group()


def test_shard_bounds_cover_the_buffer():
    for numel, world in ((64, 2), (1000, 3), (8, 8)):
        spans = [shard_bounds(numel, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == numel
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % 8 == 0 for lo, _ in spans)


@pytest.mark.timeout(300)
def test_two_gloo_ranks_match_the_replicated_optimizer(tmp_path):
    out = str(tmp_path / "r0.pt")
    port = 29600 + os.getpid() % 1000
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out)
    model = _model()
    ref = BF16Optimizer(model, lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
    for step in range(3):
        for rank in range(2):
            for p, g in zip(model.parameters(), _grads(rank, step, model)):
                p.main_grad.add_(g)
        ref.set_grad_scale(0.5)
        norm = ref.step()
    for a, b in zip(got["params"], model.parameters()):
        assert torch.allclose(a, b.detach(), atol=1e-6)
    assert torch.allclose(got["norm"], norm, rtol=1e-5)
    assert torch.allclose(got["full"][: ref.numel], ref.flat_master[: got["full"].numel()][: ref.numel], atol=1e-6)


@pytest.mark.gpu
def test_peer_memory_kernels_with_two_emulated_ranks():
    from aspec_b200.ops import comm
    from aspec_b200.ops import elementwise_sm100 as E
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    n, world = 1 << 20, 2
    grads = [torch.randn(n, device=dev) for _ in range(world)]
    w0 = torch.randn(n, device=dev)
    replicas = [w0.to(torch.bfloat16).clone() for _ in range(world)]
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.01, step=1, max_norm=0.5)
    # reference: replicated optimizer on the summed gradient
    total = grads[0] + grads[1]
    ctrl_ref = torch.zeros(4, device=dev)
    E.sumsq(total, ctrl_ref)
    ctrl_ref[2] = 0.25
    master_ref, m_ref, v_ref = w0.clone(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    param_ref = torch.empty(n, device=dev, dtype=torch.bfloat16)
    E.adamw(master_ref, total, m_ref, v_ref, param_ref, ctrl_ref, **kw)
    # sharded: phase 1 on both "ranks", the 2-float reduction, then phase 2 on both
    ctrls = [torch.zeros(4, device=dev) for _ in range(world)]
    shards = []
    for r in range(world):
        lo, hi = shard_bounds(n, r, world)
        sg = torch.empty(hi - lo, device=dev)
        comm.shard_reduce_sumsq(grads, lo, sg, ctrls[r])
        shards.append(sg)
    tot = ctrls[0][:2] + ctrls[1][:2]
    assert torch.allclose(tot[0], ctrl_ref[0], rtol=1e-4)
    for r in range(world):
        lo, hi = shard_bounds(n, r, world)
        ctrls[r][:2] = tot
        ctrls[r][2] = 0.25
        master = w0[lo:hi].clone()
        comm.shard_adamw_scatter(master, shards[r], torch.zeros(hi - lo, device=dev), torch.zeros(hi - lo, device=dev),
                                 replicas, lo, ctrls[r], **kw)
        assert torch.allclose(master, master_ref[lo:hi], atol=1e-6)
    torch.cuda.synchronize()
    for rep in replicas:
        # the two kernels may contract multiply-adds differently: masters agree to 1e-6, so at most a stray
        # round-to-bf16 differs
        assert torch.allclose(rep.float(), param_ref.float(), rtol=8e-3, atol=1e-6)
        assert (rep != param_ref).float().mean() < 1e-3
