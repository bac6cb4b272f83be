"""Grouped tcgen05 GEMM against fp32 PyTorch statements of the same products."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("b_t", [False, True])
def test_rows_gemm_with_two_sources_and_two_destinations(b_t):
    from aspec_b200.ops.gemm import check_status
    from aspec_b200.ops.grouped_gemm import rows_gemm
    E, N, K = 5, 320, 192
    a0, a1 = _bf(700, K, seed=1), _bf(500, K, seed=2)
    w = _bf(E, K, N, scale=0.1, seed=3) if b_t else _bf(E, N, K, scale=0.1, seed=3)
    src = [0, 1, 0, 1, 0, 1]
    a_row = [3, 0, 200, 130, 650, 400]
    rows = [150, 129, 0, 257, 50, 1]
    expert = [0, 1, 2, 3, 4, 2]
    dst = [0, 0, 1, 1, 0, 1]
    out_row = [0, 150, 0, 10, 300, 300]
    o0 = torch.full((400, N), 7.0, device="cuda", dtype=torch.bfloat16)
    o1 = torch.full((330, N + 64), 7.0, device="cuda", dtype=torch.bfloat16)
    rows_gemm([a0, a1], w, [o0, o1], src=src, a_row=a_row, rows=rows, expert=expert, dst=dst, out_row=out_row, b_t=b_t)
    check_status("cuda")
    e0, e1 = torch.full_like(o0, 7.0, dtype=torch.float32), torch.full_like(o1, 7.0, dtype=torch.float32)
    for s, ar, n, e, d, orow in zip(src, a_row, rows, expert, dst, out_row):
        a = (a0, a1)[s][ar:ar + n].float()
        wm = w[e].float() if b_t else w[e].float().t()
        (e0, e1)[d][orow:orow + n, :N] = a @ wm
    assert torch.allclose(o0.float(), e0, atol=0.06, rtol=0.02)
    assert torch.allclose(o1.float(), e1, atol=0.06, rtol=0.02)          # untouched rows and columns keep their 7s


def test_wgrad_gemm_reduces_over_runs_from_several_buffers():
    from aspec_b200.ops.gemm import check_status
    from aspec_b200.ops.grouped_gemm import padded_offsets, wgrad_gemm
    E, Ma, Nb = 4, 192, 320
    counts = [[70, 0, 130, 5], [1, 0, 64, 200]]                         # [source][expert]; expert 1 gets nothing
    a_bufs = [_bf(sum(c), Ma, seed=10 + i) for i, c in enumerate(counts)]   # unpadded, finite
    runs = [(s, e, counts[s][e]) for s in range(2) for e in range(E)]
    pstart, ptotal = padded_offsets([n for _, _, n in runs])
    b = torch.zeros(ptotal, Nb, device="cuda", dtype=torch.bfloat16)      # padded with zero rows
    ref = torch.zeros(E, Ma, Nb, device="cuda")
    a_row = []
    for (s, e, n), p0 in zip(runs, pstart):
        o = sum(counts[s][:e])
        a_row.append(o)
        blk = _bf(n, Nb, seed=100 + 7 * s + e) if n else torch.zeros(0, Nb, device="cuda", dtype=torch.bfloat16)
        b[p0:p0 + n] = blk
        ref[e] += a_bufs[s][o:o + n].float().t() @ blk.float()
    out = torch.full((E, Ma, Nb), 3.0, device="cuda")
    wgrad_gemm(a_bufs, [b], out, expert=[e for _, e, _ in runs], a_src=[s for s, _, _ in runs], a_row=a_row,
               b_src=[0] * len(runs), b_row=pstart, rows=[n for _, _, n in runs])
    check_status("cuda")
    assert torch.equal(out[1], torch.zeros_like(out[1]))
    assert torch.allclose(out, ref, atol=0.2, rtol=0.02)


def test_grouped_experts_match_the_per_expert_loop_forward_and_backward():
    from aspec_b200.ops.grouped_gemm import grouped_experts
    E, D, I = 6, 256, 128
    counts = [100, 0, 37, 260, 1, 64]
    x = _bf(sum(counts), D, seed=5).requires_grad_(True)
    gu = _bf(E, 2 * I, D, scale=0.05, seed=6).requires_grad_(True)
    dn = _bf(E, D, I, scale=0.05, seed=7).requires_grad_(True)
    y = grouped_experts(x, gu, dn, counts)
    dy = _bf(*y.shape, seed=8)
    y.backward(dy)
    xr, gur, dnr = (t.detach().float().requires_grad_(True) for t in (x, gu, dn))
    outs, off = [], 0
    for e, n in enumerate(counts):
        h = xr[off:off + n] @ gur[e].t()
        g, u = h[:, :I], h[:, I:]
        outs.append((torch.nn.functional.silu(g) * u) @ dnr[e].t())
        off += n
    yr = torch.cat(outs)
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, atol=0.03, rtol=0.03)
    assert torch.allclose(x.grad.float(), xr.grad, atol=0.03, rtol=0.05)
    assert torch.allclose(gu.grad.float(), gur.grad, atol=0.15, rtol=0.05)
    assert torch.allclose(dn.grad.float(), dnr.grad, atol=0.15, rtol=0.05)


def test_eagle4_swiglu_moe_runs_on_the_grouped_kernels_and_matches_fp32():
    """The EAGLE4 mixture-of-experts block: bf16 on the GPU (grouped launches) against the same module in fp32 on the CPU."""
    from types import SimpleNamespace
    from aspec_b200.models.draft.eagle4_moe import Eagle4MoE
    cfg = SimpleNamespace(hidden_size=128, moe_intermediate_size=64, n_routed_experts=8, num_experts_per_tok=2, hidden_act="silu",
                          n_group=2, topk_group=1, norm_topk_prob=True, routed_scaling_factor=1.5, n_shared_experts=1,
                          moe_architecture="sparse_swiglu", initializer_range=0.05)
    torch.manual_seed(0)
    ref = Eagle4MoE(cfg)
    with torch.no_grad():
        ref.experts["w2_weight"].normal_(std=0.05)              # the bank starts as a no-op: give it something to compute
    gpu = Eagle4MoE(cfg)
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.to("cuda", torch.bfloat16)
    x = torch.randn(300, 128) * 0.5
    xg = x.to("cuda", torch.bfloat16).requires_grad_(True)
    xr = x.bfloat16().float().requires_grad_(True)
    yg = gpu(xg)
    yr = ref(xr)
    dy = torch.randn(300, 128) * 0.1
    yg.backward(dy.to("cuda", torch.bfloat16))
    yr.backward(dy.bfloat16().float())
    assert torch.allclose(yg.float().cpu(), yr, atol=0.05, rtol=0.05)
    assert torch.allclose(xg.grad.float().cpu(), xr.grad, atol=0.05, rtol=0.1)
    w13_g, w13_r = gpu.experts["w13_weight"].grad.float().cpu(), ref.experts["w13_weight"].grad
    assert torch.allclose(w13_g, w13_r, atol=0.05 * max(w13_r.abs().max().item(), 1e-3) + 0.02, rtol=0.1)
