"""Small single-kernel workloads for profiler captures: ``python -m tools.performance.profile_cases CASE``.

Each case launches its kernel a few times on inputs larger than the 126 MB L2 but well under a few GB, so
that ``ncu --set full --clock-control none -k regex:<kernel> -c 1..3`` finishes in about a minute.  The flag
``--clock-control none`` matters on shared GPUs: without it the profiler locks the clocks and a killed capture can
leave them locked for the next user.  Capture one kernel on these small cases only, after the same command line has
run to completion without the profiler.  Cases: ``gemm``, ``gemm_head``,
``attn_fwd``, ``attn_bwd``, ``vocab_loss``, ``rmsnorm``, ``grouped_experts``, ``sel_attn`` (selected-key attention
forward + backward), ``indexer`` (scores + top-k), and the compute+collective kernels with every "peer" buffer placed on
this same GPU - ``gemm_mirror`` (GEMM whose epilogue also stores the tile into two more destinations), ``gemm_scatter``
(column-scatter epilogue of the Ulysses projection), ``shard_step`` (peer-sum of gradient shards + sum of squares, then
AdamW with the bf16 weights stored into every replica), ``peer_lse`` (log-sum-exp merge over peers' statistics), ``full_shard`` (a layer's parameter
gather and gradient reduce-scatter of the FULL_SHARD strategy).  On one
GPU these captures show the kernels' DRAM and tensor-pipe behaviour; NVLink traffic is by construction zero here.
"""
from __future__ import annotations

import sys

import torch


def _bf16(*shape, scale=0.05):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def case_gemm():
    from aspec_b200.ops import gemm as G
    a, b = _bf16(8192, 4096), _bf16(8192, 4096)
    out = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        G.gemm(a, b, out=out)


def case_gemm_head():
    from aspec_b200.ops import gemm as G
    a, b = _bf16(3584, 4096), _bf16(32768, 4096)
    stats = torch.empty(128, 3584, 2, device="cuda")
    out = torch.empty(3584, 32768, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        G.gemm(a, b, out=out, epilogue=G.EPI_ROWSTATS, stats=stats)


def _attn_inputs(n_ctx=16384, n_blocks=1024, bs=7, hq=32, hkv=8):
    from aspec_b200.ops.attention import build_block_intervals
    g = torch.Generator().manual_seed(0)
    anchors = torch.sort(torch.randint(1, n_ctx - bs, (n_blocks,), generator=g)).values
    iv = build_block_intervals(anchors, torch.ones(n_blocks, dtype=torch.bool), ctx_len=n_ctx, block_size=bs).cuda()
    Q = n_blocks * bs
    return _bf16(Q, hq, 128, scale=1.0), _bf16(n_ctx + Q, hkv, 128, scale=1.0), _bf16(n_ctx + Q, hkv, 128, scale=1.0), iv


def case_attn_fwd():
    from aspec_b200.ops import attention_sm100 as A
    q, k, v, iv = _attn_inputs()
    for _ in range(3):
        A.forward(q, k, v, iv, 128 ** -0.5)


def case_attn_bwd():
    from aspec_b200.ops import attention_sm100 as A
    q, k, v, iv = _attn_inputs()
    out, lse = A.forward(q, k, v, iv, 128 ** -0.5)
    do = torch.randn_like(out)
    for _ in range(2):
        A.backward(q, k, v, iv, out, lse, do, 128 ** -0.5)


def case_grouped_experts():
    from aspec_b200.ops.grouped_gemm import grouped_experts
    E, D, I, N = 64, 2048, 1024, 32768
    g = torch.Generator().manual_seed(0)
    counts = torch.bincount(torch.randint(0, E, (N,), generator=g), minlength=E).tolist()
    x, gu, dn = _bf16(N, D, scale=1.0), _bf16(E, 2 * I, D), _bf16(E, D, I)
    for _ in range(3):
        grouped_experts(x, gu, dn, counts)


def case_vocab_loss():
    from aspec_b200.ops import elementwise_sm100 as E
    R, V = 1792, 151936
    s, t = _bf16(R, V, scale=1.0), _bf16(R, V, scale=1.0)
    lse = torch.logsumexp(s.float(), -1)
    lse_t = torch.logsumexp(t.float(), -1)
    labels = torch.randint(0, V, (R,), device="cuda")
    w = torch.rand(R, device="cuda")
    idx = torch.arange(R, device="cuda", dtype=torch.int32)
    for _ in range(2):
        E.vocab_loss(s, t, lse, lse_t, idx, labels, w, mode=0, a_ce=0.1, a_l1=0.9, write_grad=True)


def case_rmsnorm():
    from aspec_b200.ops import elementwise_sm100 as E
    x, w = _bf16(32768, 4096, scale=1.0), _bf16(4096, scale=1.0)
    for _ in range(3):
        E.rmsnorm_fwd(x, w, 1e-6)


def case_sel_attn():
    from aspec_b200.ops import sparse_attention as SA
    n, T, L, hq, hkv = 1024, 65536, 1024 + 7, 32, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (_bf16(n, hq, 128, scale=1.0).requires_grad_(), _bf16(T, hkv, 128, scale=1.0).requires_grad_(),
               _bf16(T, hkv, 128, scale=1.0).requires_grad_())
    sel = torch.randint(0, T, (n, L), generator=g).to(torch.int32).cuda()
    for _ in range(2):
        out, _ = SA.selected_attention(q, k, v, sel, 128 ** -0.5)
        out.backward(torch.ones_like(out))


def case_indexer():
    from aspec_b200.ops import sparse_attention as SA
    n, T, H, d = 256, 16384, 64, 128
    qi, ki = _bf16(n, H, d, scale=1.0), _bf16(T, d, scale=1.0)
    w = torch.rand(n, H, device="cuda") * 0.1
    lo = torch.zeros(n, dtype=torch.int32, device="cuda")
    hi = torch.randint(T // 2, T, (n,), device="cuda").to(torch.int32)
    for _ in range(2):
        s = SA.indexer_scores(qi, ki, w, lo, hi)
        SA.topk_select(s, lo, hi, 1024)


def case_gemm_mirror():
    from aspec_b200.ops import gemm as G
    a, b = _bf16(8192, 4096), _bf16(4096, 4096)
    out = torch.empty(8192, 4096, device="cuda", dtype=torch.bfloat16)
    mirrors = [torch.empty_like(out), torch.empty_like(out)]
    for _ in range(3):
        G.gemm(a, b, out=out, mirrors=mirrors)


def case_gemm_scatter():
    from aspec_b200.ops import gemm as G
    a, b = _bf16(8192, 4096), _bf16(6144, 4096)
    dests = [torch.empty(8192, 6144 // 4, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    for _ in range(3):
        G.gemm(a, b, mirrors=dests, scatter_cols=6144 // 4)


def case_shard_step():
    from aspec_b200.ops import comm
    n, peers = 64 << 20, 4
    grads = [torch.randn(n, device="cuda") for _ in range(peers)]
    params = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(peers)]
    shard, master, m, v = (torch.zeros(n, device="cuda") for _ in range(4))
    ctrl = torch.zeros(8, device="cuda")
    for _ in range(2):
        ctrl.zero_()
        comm.shard_reduce_sumsq(grads, 0, shard, ctrl)
        ctrl[2] = 1.0
        ctrl[4] = 1.0
        comm.shard_adamw_scatter(master, shard, m, v, params, 0, ctrl, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0,
                                 step=None, max_norm=1.0)


def case_peer_lse():
    from aspec_b200.ops import comm
    n, peers = 32 << 20, 8
    parts = [torch.randn(n, device="cuda") for _ in range(peers)]
    out = torch.empty(n, device="cuda")
    for _ in range(3):
        comm.peer_lse_merge(parts, out)


def case_full_shard():
    """The two data kernels of FULL_SHARD with four ranks' buffers on one device: a layer's parameter gather
    (4 x 64 MB bf16 shards -> one 256 MB working copy) and its gradient reduce-scatter (this rank's quarter of four
    512 MB fp32 replicas, accumulated into the shard)."""
    from aspec_b200.ops import comm
    per, peers = 32 << 20, 4
    shards = [torch.randn(per, device="cuda").bfloat16() for _ in range(peers)]
    whole = torch.empty(per * peers, device="cuda", dtype=torch.bfloat16)
    grads = [torch.randn(per * peers, device="cuda") for _ in range(peers)]
    mine = torch.zeros(per, device="cuda")
    for _ in range(3):
        comm.peer_gather(shards, whole)
        comm.shard_reduce_accum(grads, per, mine)


CASES = {n[5:]: f for n, f in globals().items() if n.startswith("case_")}

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    CASES[name]()
    torch.cuda.synchronize()
    from aspec_b200.ops.gemm import check_status
    check_status("cuda")
    print("ok", name)
