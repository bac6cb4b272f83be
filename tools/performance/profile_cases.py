"""Small single-kernel workloads for profiler captures: ``python -m tools.performance.profile_cases CASE``.

Each case launches its kernel a few times on inputs larger than the 126 MB L2 but well under a few GB, so
that ``ncu --set full --clock-control none -k regex:<kernel> -c 1..3`` finishes in about a minute.  The flag
``--clock-control none`` matters on shared GPUs: without it the profiler locks the clocks and a killed capture can
leave them locked for the next user.  Capture one kernel on these small cases only, after the same command line has
run to completion without the profiler.  Cases: ``gemm``, ``gemm_head``,
``attn_fwd``, ``attn_bwd``, ``vocab_loss``, ``rmsnorm``, ``grouped_experts``.
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


CASES = {n[5:]: f for n, f in globals().items() if n.startswith("case_")}

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    CASES[name]()
    torch.cuda.synchronize()
    from aspec_b200.ops.gemm import check_status
    check_status("cuda")
    print("ok", name)
