"""Micro-benchmarks of the peer-memory parallel layers against their library-collective baselines.

Run with one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m tools.performance.bench_parallel [--cases fsdp,vocab,cp,ulysses] [--iters 20]

Every case is timed with CUDA events on the launching stream after warm-up, a barrier and a synchronize on both
sides; the reported time is the maximum over ranks.  Between iterations a buffer larger than L2 is written.  Rank 0
prints one JSON line per case with the fused time, the baseline time (same math, NCCL collectives for the data
movement) and the roofline terms: bytes that must cross NVLink per rank and FLOPs per rank.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0          # measured peer copy bandwidth per direction per GPU on this pool
PEAK_TFLOPS = 1590.0        # fallback burst cuBLAS bf16; replaced by the measured file when present


def _peak() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["bf16_tflops"])
    except Exception:                                            # noqa: BLE001 - fall back to the stated figure
        return PEAK_TFLOPS


class Timer:
    def __init__(self, dev, iters: int, warmup: int = 3):
        self.dev, self.iters, self.warmup = dev, iters, warmup
        self.flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        total = 0.0
        for _ in range(self.iters):
            self.flush.add_(1)                       # evict L2
            dist.barrier()
            torch.cuda.synchronize(self.dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(self.dev)
            total += e0.elapsed_time(e1)
        t = torch.tensor([total / self.iters], device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)


def case_fsdp(rank, world, dev, timer, barrier):
    from aspec_b200.ops import comm
    from aspec_b200.ops import elementwise_sm100 as E
    from aspec_b200.parallel.symmetric_memory import SymmetricBuffer
    from aspec_b200.training.sharded_optimizer import shard_bounds
    n = 256 * 1024 * 1024 // 8 * 8                      # 268 M parameters (one Qwen3-8B-shaped draft layer + heads)
    pm, gm = SymmetricBuffer.allocate(n * 2, dev), SymmetricBuffer.allocate(n * 4, dev)
    param, grad = pm.tensor.view(torch.bfloat16), gm.tensor.view(torch.float32)
    grad.normal_()
    metas = [{"p": pm.export(), "g": gm.export()} for _ in range(world)]
    got = [None] * world
    dist.all_gather_object(got, metas)
    opened = [None if r == rank else (SymmetricBuffer.open(got[r][rank]["p"]), SymmetricBuffer.open(got[r][rank]["g"])) for r in range(world)]
    params = [param if r == rank else opened[r][0].tensor.view(torch.bfloat16) for r in range(world)]
    grads = [grad if r == rank else opened[r][1].tensor.view(torch.float32) for r in range(world)]
    lo, hi = shard_bounds(n, rank, world)
    own = hi - lo
    sg, ms, m, v = (torch.zeros(own, device=dev) for _ in range(4))
    ctrl = torch.zeros(4, device=dev)
    kw = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, step=1, max_norm=0.5)

    def fused():
        ctrl.zero_()
        barrier()
        comm.shard_reduce_sumsq(grads, lo, sg, ctrl)
        dist.all_reduce(ctrl[0:2])
        ctrl[2] = 1.0
        comm.shard_adamw_scatter(ms, sg, m, v, params, lo, ctrl, **kw)
        barrier()

    full_m, full_mm, full_v = (torch.zeros(n, device=dev) for _ in range(3))
    rgrad = torch.randn(n, device=dev)

    def replicated():                                  # all-reduce + replicated update (the REPLICATE strategy)
        ctrl.zero_()
        dist.all_reduce(rgrad)
        E.sumsq(rgrad, ctrl)
        ctrl[2] = 1.0
        E.adamw(full_m, rgrad, full_mm, full_v, param, ctrl, **kw)

    per = shard_bounds(n, 0, world)[1]
    rs_out = torch.zeros(per, device=dev)
    ag_in = torch.zeros(per, device=dev, dtype=torch.bfloat16)
    ag_out = torch.zeros(per * world, device=dev, dtype=torch.bfloat16)
    rs_in = torch.randn(per * world, device=dev)

    def library_sharded():                             # reduce-scatter + sharded update + all-gather through NCCL
        ctrl.zero_()
        dist.reduce_scatter_tensor(rs_out, rs_in)
        E.sumsq(rs_out[:own], ctrl)
        dist.all_reduce(ctrl[0:2])
        ctrl[2] = 1.0
        E.adamw(ms, rs_out[:own], m, v, ag_in[:own], ctrl, **kw)
        dist.all_gather_into_tensor(ag_out, ag_in)

    t_f, t_r, t_l = timer(fused), timer(replicated), timer(library_sharded)
    nv_bytes = (world - 1) * own * 4 + (world - 1) * own * 2          # pulled gradients + pushed weights, per rank
    return {"case": "fsdp_sharded_adamw", "params": n, "fused_ms": t_f, "nccl_allreduce_replicated_ms": t_r,
            "nccl_reduce_scatter_all_gather_ms": t_l, "nvlink_bytes_per_rank": nv_bytes,
            "nvlink_floor_ms": nv_bytes / (NVLINK_GBS * 1e6), "achieved_over_floor": (nv_bytes / (NVLINK_GBS * 1e6)) / t_f,
            "optimizer_state_bytes_per_rank": own * 12, "replicated_state_bytes": n * 12}


def case_vocab(rank, world, dev, timer, barrier):
    from aspec_b200.ops.vocab_head import head_loss
    from aspec_b200.parallel.group import exchange_workspaces
    from aspec_b200.parallel.vocab_parallel import VocabParallelHead, VocabShardWorkspace, vocab_parallel_head_loss
    bf = torch.bfloat16
    R, Tt, D, V, rk = 3584, 1536, 4096, 151936, 256
    torch.manual_seed(0)
    hidden = (torch.randn(R, D, device=dev) * 0.5).to(bf)
    W = (torch.randn(V, D, device=dev) * 0.02).to(bf)
    W2 = (torch.randn(V, rk, device=dev) * 0.02).to(bf)
    prev = (torch.randn(R, rk, device=dev) * 0.5).to(bf)
    teacher = (torch.randn(Tt, D, device=dev) * 0.5).to(bf)
    t_index = torch.randint(0, Tt, (R,), device=dev, dtype=torch.int32)
    labels = torch.randint(0, V, (R,), device=dev)
    weight = torch.rand(R, device=dev)
    ws = exchange_workspaces(VocabShardWorkspace(R, Tt, D, rk, world, device=dev), VocabShardWorkspace.open)
    head = VocabParallelHead(rank, world, V, ws, barrier)
    Ws = head.shard_rows(W).contiguous()

    def replicated():
        h, p = hidden.clone().requires_grad_(True), prev.clone().requires_grad_(True)
        num, *_ = head_loss(h, W, labels, weight, prev_emb=p, markov_w2=W2, teacher_hidden=teacher, t_index=t_index, a_ce=0.1, a_l1=0.9)
        num.backward()

    def sharded():
        h, p = hidden.clone().requires_grad_(True), prev.clone().requires_grad_(True)
        num, *_ = vocab_parallel_head_loss(head, h, Ws, labels, weight, prev_emb=p, markov_w2=W2, teacher_hidden=teacher,
                                           t_index=t_index, a_ce=0.1, a_l1=0.9)
        num.backward()

    t_s, t_r = timer(sharded), timer(replicated)
    flops = 2.0 * V / world * (D + rk) * (2 * R + Tt) + 2.0 * V / world * rk * R
    nv = (world - 1) * R * (D + rk) * 2
    floor = max(flops / (_peak() * 1e9), nv / (NVLINK_GBS * 1e6))
    return {"case": "vocab_parallel_head", "rows": R, "vocab": V, "sharded_ms": t_s, "replicated_head_ms": t_r,
            "flops_per_rank": flops, "nvlink_bytes_per_rank": nv, "roofline_ms": floor, "achieved_over_roofline": floor / t_s,
            "head_weight_bytes_per_rank": V // world * (D + rk) * 2}


def case_cp(rank, world, dev, timer, barrier):
    from aspec_b200.ops import attention_sm100 as K
    from aspec_b200.ops.attention import build_block_intervals, merge_partials
    from aspec_b200.parallel.context import context_shard_bounds
    from aspec_b200.parallel.context_parallel import CPWorkspace, DirectCPAttention, local_intervals
    from aspec_b200.parallel.group import exchange_workspaces
    bf = torch.bfloat16
    T, A, bs, H, Hk, d = 131072, 512 * world, 7, 32, 8, 128
    Q = A * bs
    ql = Q // world
    torch.manual_seed(0)
    anchors = torch.sort(torch.randint(64, T - bs, (A,), device=dev)).values
    dist.broadcast(anchors, 0)
    iv = build_block_intervals(anchors, torch.ones(A, dtype=torch.bool, device=dev), ctx_len=T, block_size=bs)
    s, e = context_shard_bounds(T, rank, world, 1)
    k_loc = (torch.randn(e - s + ql, Hk, d, device=dev) * 0.5).to(bf)
    v_loc = (torch.randn(e - s + ql, Hk, d, device=dev) * 0.5).to(bf)
    q_loc = (torch.randn(ql, H, d, device=dev) * 0.5).to(bf)
    dout = (torch.randn(ql, H, d, device=dev) * 0.5).to(bf)
    tables = [local_intervals(iv[o * ql:(o + 1) * ql], s, e, T, own=(o == rank), query_start=rank * ql) for o in range(world)]
    ws = exchange_workspaces(CPWorkspace(world, ql, H, d, device=dev), CPWorkspace.open)
    cp = DirectCPAttention(rank, world, ws, barrier)
    scale = d ** -0.5

    def fused():
        cp.publish(q_loc)
        barrier()
        cp.partials(k_loc, v_loc, tables, [ql] * world, scale)
        barrier()
        cp.merge()
        barrier()
        cp.publish_grad(dout)
        barrier()
        cp.grad_partials()
        barrier()
        cp.reduce_grad()
        barrier()

    q_all = torch.empty(Q, H, d, device=dev, dtype=bf)
    table_all = torch.cat(tables)
    po = torch.empty(world, ql, H, d, device=dev, dtype=bf)
    pl = torch.empty(world, H, ql, device=dev)

    def library():                                   # all-gather Q, partial attention, all-to-all partials, merge; same for backward
        dist.all_gather_into_tensor(q_all, q_loc)
        o, l = K.forward(q_all, k_loc, v_loc, table_all, scale)
        dist.all_to_all_single(po, o.view(world, ql, H, d))
        dist.all_to_all_single(pl, l.view(H, world, ql).permute(1, 0, 2).contiguous())
        om, lm = merge_partials(po, pl)
        o_all, l_all, d_all = torch.empty_like(q_all), torch.empty(world, H, ql, device=dev), torch.empty_like(q_all)
        dist.all_gather_into_tensor(o_all, om)
        dist.all_gather_into_tensor(l_all, lm)
        dist.all_gather_into_tensor(d_all, dout)
        dq, _dk, _dv = K.backward(q_all, k_loc, v_loc, table_all, o_all, l_all.permute(1, 0, 2).reshape(H, Q).contiguous(), d_all, scale)
        out = torch.empty(ql, H, d, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(out, dq.float())

    t_f, t_l = timer(fused), timer(library)
    return {"case": "direct_cp_attention_fwd_bwd", "context": T, "queries": Q, "fused_ms": t_f, "nccl_gather_a2a_ms": t_l,
            "nvlink_bytes_per_rank": (world - 1) * ql * H * d * 2 * 6}


def case_ulysses(rank, world, dev, timer, barrier):
    from aspec_b200.ops import gemm as G
    from aspec_b200.parallel.group import exchange_workspaces
    from aspec_b200.parallel.ulysses import UlyssesExchange, UlyssesWorkspace
    bf = torch.bfloat16
    T_loc, D, hq, hk, d = 16384 // world, 4096, 32, 8, 128
    qc, oc = (hq + 2 * hk) * d // world, hq * d // world
    x = (torch.randn(T_loc, D, device=dev) * 0.5).to(bf)
    wg = (torch.randn((hq + 2 * hk) * d, D, device=dev) * 0.02).to(bf)
    wo = (torch.randn(D, hq * d, device=dev) * 0.02).to(bf)
    ws = exchange_workspaces(UlyssesWorkspace(world, T_loc, qc, oc, device=dev), UlyssesWorkspace.open)
    ex = UlyssesExchange(rank, world, ws, barrier)
    ex.mine.attn.normal_()

    def fused():
        ex.project_scatter(x, wg)
        barrier()
        ex.output_projection(wo)
        barrier()

    recv = torch.empty(world, T_loc, qc, device=dev, dtype=bf)
    attn = torch.randn(world * T_loc, oc, device=dev).to(bf)
    back = torch.empty(world, T_loc, oc, device=dev, dtype=bf)

    def library():
        qkv = G.gemm(x, wg)
        dist.all_to_all_single(recv, qkv.view(T_loc, world, qc).permute(1, 0, 2).contiguous())
        dist.all_to_all_single(back, attn.view(world, T_loc, oc))
        G.gemm(back.permute(1, 0, 2).reshape(T_loc, hq * d), wo)

    t_f, t_l = timer(fused), timer(library)
    flops = 2.0 * T_loc * D * ((hq + 2 * hk) * d + hq * d)
    nv = (world - 1) * T_loc * (qc + oc) * 2
    floor = max(flops / (_peak() * 1e9), nv / (NVLINK_GBS * 1e6))
    return {"case": "ulysses_projections", "rows_per_rank": T_loc, "fused_ms": t_f, "gemm_plus_nccl_a2a_ms": t_l,
            "flops_per_rank": flops, "nvlink_bytes_per_rank": nv, "roofline_ms": floor, "achieved_over_roofline": floor / t_f}


def case_moe(rank, world, dev, timer, barrier):
    from aspec_b200.models.draft.moe import ExpertBank
    from aspec_b200.parallel.expert_parallel import (EPWorkspace, FusedExpertParallel, dispatch_combine, exchange_counts,
                                                     fused_dispatch_combine)
    from aspec_b200.parallel.group import exchange_workspaces
    bf = torch.bfloat16
    E, D, I, N, k = 64, 2048, 1024, 3584, 4               # Ling-flash-like block: 3584 supervised rows, top-4 of 64
    bank = ExpertBank(E, D, I, ep_rank=rank, ep_size=world).to(dev, bf)
    torch.manual_seed(rank)
    x = (torch.randn(N, D, device=dev) * 0.5).to(bf)
    sel = torch.randint(0, E, (N * k,), device=dev)
    order = torch.argsort(sel, stable=True)
    xs = x.repeat_interleave(k, 0)[order].contiguous()
    se = sel[order]
    dy = (torch.randn(N * k, D, device=dev) * 0.1).to(bf)
    ws = exchange_workspaces(EPWorkspace(N * k, D, device=dev), EPWorkspace.open)
    ep = FusedExpertParallel(rank, world, E, ws, barrier)

    def fused():
        a = xs.clone().requires_grad_(True)
        fused_dispatch_combine(ep, bank, a, se).backward(dy)

    def library():
        a = xs.clone().requires_grad_(True)
        dispatch_combine(bank, a, se).backward(dy)

    t_f, t_l = timer(fused), timer(library)
    rows_remote = N * k * (world - 1) / world
    flops = 3 * 2.0 * N * k * D * 3 * I                     # fwd + dgrad + wgrad of the two GEMMs (gate/up is 2I wide)
    nv = rows_remote * D * 2 * 4                            # x, y, dy, dx rows that belong to remote experts
    floor = max(flops / (_peak() * 1e9), nv / (NVLINK_GBS * 1e6))
    return {"case": "moe_expert_parallel_fwd_bwd", "rows": N * k, "experts": E, "fused_ms": t_f, "nccl_all_to_all_ms": t_l,
            "flops_per_rank": flops, "nvlink_bytes_per_rank": nv, "roofline_ms": floor, "achieved_over_roofline": floor / t_f}


CASES = {"moe": case_moe, "fsdp": case_fsdp, "vocab": case_vocab, "cp": case_cp, "ulysses": case_ulysses}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="fsdp,vocab,cp,ulysses,moe")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from aspec_b200.parallel.group import make_barrier
    barrier = make_barrier(dev)
    timer = Timer(dev, a.iters)
    for name in a.cases.split(","):
        try:
            res = CASES[name](rank, world, dev, timer, barrier)
        except Exception as exc:                                 # noqa: BLE001 - one case must not hide the others
            res = {"case": name, "error": f"{type(exc).__name__}: {exc}"}
        res["n_gpus"] = world
        if rank == 0:
            print(json.dumps(res), flush=True)
        torch.cuda.empty_cache()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
