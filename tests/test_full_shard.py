"""FULL_SHARD (parameters, gradients and optimizer state sharded per layer): the protocol must train exactly like the
replicated optimizer.  CPU: two and three gloo ranks through real forward / backward passes with two micro-batches.
GPU: the kernel path on one rank, and the gather / reduce / flag kernels over two emulated ranks' buffers."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch.utils.checkpoint import checkpoint

from aspec_b200.training.full_shard import FullShardOptimizer
from aspec_b200.training.optimizer import BF16Optimizer


class _Layer(torch.nn.Module):
    def __init__(self, d):
        super().__init__()
        self.a = torch.nn.Linear(d, d, bias=False)
        self.b = torch.nn.Linear(d, d, bias=True)
        self.c = torch.nn.Linear(d, d, bias=False)

    def forward(self, x, ctx, scale):
        return x + torch.tanh(self.a(x) + self.b(ctx)) * scale, self.c(ctx).mean()


class _Net(torch.nn.Module):
    """A frozen embedding feeds x (no gradient into layer 0 through x); ``inp`` makes ctx differentiable."""

    def __init__(self, d=12, layers=3, ckpt=False):
        super().__init__()
        self.embed = torch.nn.Embedding(50, d)
        self.embed.weight.requires_grad_(False)
        self.inp = torch.nn.Linear(7, d, bias=False)
        self.layers = torch.nn.ModuleList([_Layer(d) for _ in range(layers)])
        self.out = torch.nn.Linear(d, 5, bias=False)
        self.ckpt = ckpt

    def forward(self, ids, feats):
        x, ctx = self.embed(ids), self.inp(feats)
        extra = 0.0
        for i, layer in enumerate(self.layers):
            if self.ckpt and i == 1:
                x, e = checkpoint(layer, x, ctx, 0.5, use_reentrant=False)
            else:
                x, e = layer(x, ctx, 0.5)
            extra = extra + e
        return self.out(x).pow(2).mean() + 0.1 * extra


def _data(rank, step, mb):
    g = torch.Generator().manual_seed(1000 * step + 10 * rank + mb)
    return torch.randint(0, 50, (9,), generator=g), torch.randn(9, 7, generator=g)


def _net(ckpt):
    torch.manual_seed(3)
    return _Net(ckpt=ckpt)


def _units(net, wrap):
    """``wrap=False``: no module is a unit of its own (a Draft whose decoder is not a ``layers`` list): all in the root."""
    return list(net.layers) if wrap else []


def _worker(rank, world, port, out, ckpt, wrap=True):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    net = _net(ckpt)
    opt = FullShardOptimizer(net, _units(net, wrap), lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
    report = opt.memory_report()
    norms = []
    for step in range(3):
        for mb in range(2):
            net(*_data(rank, step, mb)).backward()
            opt.finish_micro_batch()
        opt.set_grad_scale(0.25)
        norms.append(opt.step())
    state = opt.state_dict()
    with opt.full_parameters():
        params = {n: p.detach().clone() for n, p in net.named_parameters()}
    # a second optimizer restored from the state continues identically
    net2 = _net(ckpt)
    opt2 = FullShardOptimizer(net2, _units(net2, wrap), lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
    opt2.load_state_dict(state)
    opt2.scheduler.load_state_dict(opt.scheduler.state_dict())
    for o, n in ((opt, net), (opt2, net2)):
        n(*_data(rank, 9, 0)).backward()
        o.finish_micro_batch()
        o.step()
    with opt.full_parameters():
        cont_a = [p.detach().clone() for p in net.parameters()]
    with opt2.full_parameters():
        cont_b = [p.detach().clone() for p in net2.parameters()]
    if rank == 0:
        torch.save({"params": params, "norms": norms, "report": report, "master": state["master"],
                    "resume_equal": all(torch.equal(a, b) for a, b in zip(cont_a, cont_b))}, out)
    dist.destroy_process_group()


def _replicated(world, ckpt):
    net = _net(ckpt)
    ref = BF16Optimizer(net, lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
    norms = []
    for step in range(3):
        for rank in range(world):
            for mb in range(2):
                net(*_data(rank, step, mb)).backward()
        ref.set_grad_scale(0.25)
        norms.append(ref.step())
    return net, ref, norms


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world,ckpt,wrap", [(2, False, True), (3, True, True), (2, False, False)])
def test_gloo_ranks_train_like_the_replicated_optimizer(tmp_path, world, ckpt, wrap):
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, 29700 + os.getpid() % 500 + world, out, ckpt, wrap), nprocs=world, join=True)
    got = torch.load(out)
    net, ref, norms = _replicated(world, ckpt)
    for a, b in zip(got["norms"], norms):
        assert torch.allclose(a, b, rtol=1e-5)
    for name, p in net.named_parameters():
        assert torch.allclose(got["params"][name], p.detach(), atol=1e-6), name
    for name, m in ref.state_dict()["master"].items():
        assert torch.allclose(got["master"][name], m, atol=1e-6), name
    assert got["resume_equal"]
    rep = got["report"]
    assert rep["world"] == world and rep["at_rest_bytes"] * world <= rep["replicated_bytes"] * 1.2 + 4096
    if wrap:
        assert rep["working_bytes"] < rep["replicated_bytes"]      # two layers + root of working copies, not the model


def test_single_rank_is_the_plain_optimizer():
    net_a, net_b = _net(False), _net(False)
    a = FullShardOptimizer(net_a, list(net_a.layers), lr=1e-2, max_grad_norm=0.5, total_steps=50)
    b = BF16Optimizer(net_b, lr=1e-2, max_grad_norm=0.5, total_steps=50)
    for step in range(2):
        net_a(*_data(0, step, 0)).backward()
        a.finish_micro_batch()
        net_b(*_data(0, step, 0)).backward()
        na, nb = a.step(), b.step()
        assert torch.allclose(na, nb, rtol=1e-6)
    with a.full_parameters():
        for p, q in zip(net_a.parameters(), net_b.parameters()):
            assert torch.allclose(p, q, atol=1e-7)
    # loading weights through the writeback block re-seeds shards and masters
    with a.full_parameters(writeback=True):
        for p in net_a.parameters():
            if p.requires_grad:
                p.data.fill_(0.25)
    u0 = a.units[0]
    n0 = u0.params[0].numel()
    assert torch.all(a.shard_master[u0.shard_offset:u0.shard_offset + n0] == 0.25)
    with a.full_parameters():
        assert all(torch.all(p == 0.25) for p in net_a.parameters() if p.requires_grad)
    with torch.no_grad():
        assert torch.isfinite(net_a(*_data(0, 0, 0)))


@pytest.mark.gpu
def test_kernel_path_on_one_rank_and_the_collective_kernels_over_two_emulated_ranks():
    from aspec_b200.ops import comm
    dev = torch.device("cuda:0")
    net_a, net_b = _net(False).to(dev, torch.bfloat16), _net(False).to(dev, torch.bfloat16)
    a = FullShardOptimizer(net_a, list(net_a.layers), lr=1e-2, max_grad_norm=0.5, total_steps=50)
    b = BF16Optimizer(net_b, lr=1e-2, max_grad_norm=0.5, total_steps=50)
    assert a.use_kernel
    for step in range(2):
        for mb in range(2):
            ids, feats = _data(0, step, mb)
            net_a(ids.to(dev), feats.to(dev, torch.bfloat16)).backward()
            a.finish_micro_batch()
            net_b(ids.to(dev), feats.to(dev, torch.bfloat16)).backward()
        na, nb = a.step(), b.step()
        assert torch.allclose(na, nb, rtol=2e-2)
    with a.full_parameters():
        for p, q in zip(net_a.parameters(), net_b.parameters()):
            assert torch.allclose(p.float(), q.float(), atol=2e-2)
    # gather: two "ranks'" shards -> one whole buffer
    shards = [torch.randn(4096, device=dev).bfloat16() for _ in range(2)]
    whole = torch.empty(8192, device=dev, dtype=torch.bfloat16)
    comm.peer_gather(shards, whole)
    assert torch.equal(whole, torch.cat(shards))
    # reduce-scatter with accumulation: rank 1's range of two replicas
    grads = [torch.randn(8192, device=dev) for _ in range(2)]
    mine = torch.ones(4096, device=dev)
    comm.shard_reduce_accum(grads, 4096, mine)
    assert torch.allclose(mine, 1.0 + grads[0][4096:] + grads[1][4096:], atol=1e-6)
    # flags: a value published to both arrays passes the wait; a value nobody publishes runs the bounded wait out
    flags = [torch.zeros(14, dtype=torch.int64, device=dev) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    comm.flags_signal(flags, 2 * 2 + 0, 5)           # slot 2, writer 0
    comm.flags_signal(flags, 2 * 2 + 1, 5)           # slot 2, writer 1
    comm.flags_wait_all(flags[1], 2 * 2, 2, 5, status, limit_ms=2000.0)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and flags[0][4:6].tolist() == [5, 5]
    comm.flags_wait_all(flags[1], 3 * 2, 2, 1, status, limit_ms=5.0)
    torch.cuda.synchronize()
    assert int(status.item()) != 0
    assert torch.equal(whole, torch.cat(shards))     # the context is alive after the timeout
