"""Direct context-parallel attention with two ranks emulated on one GPU (phases interleaved) against single-device
interval attention on the full key set."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_emulated_ranks_match_single_device_attention():
    from aspec_b200.ops import attention_sm100 as K
    from aspec_b200.ops.attention import build_block_intervals
    from aspec_b200.parallel.context import context_shard_bounds
    from aspec_b200.parallel.context_parallel import CPWorkspace, DirectCPAttention, local_intervals
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    T, A, bs, H, Hk, d, world = 600, 32, 4, 8, 2, 128, 2
    Q = A * bs
    anchors = torch.sort(torch.randint(8, T - bs, (A,), device=dev)).values
    iv = build_block_intervals(anchors, torch.ones(A, dtype=torch.bool, device=dev), ctx_len=T, block_size=bs)
    bf = torch.bfloat16
    q = (torch.randn(Q, H, d, device=dev) * 0.5).to(bf)
    k = (torch.randn(T + Q, Hk, d, device=dev) * 0.5).to(bf)
    v = (torch.randn(T + Q, Hk, d, device=dev) * 0.5).to(bf)
    dout = (torch.randn(Q, H, d, device=dev) * 0.5).to(bf)
    scale = d ** -0.5
    out_ref, lse_ref = K.forward(q, k, v, iv, scale)
    dq_ref, dk_ref, dv_ref = K.backward(q, k, v, iv, out_ref, lse_ref, dout, scale)
    # two ranks: contiguous context ownership, contiguous query ownership
    ql = Q // world
    bounds = [context_shard_bounds(T, r, world, 1) for r in range(world)]
    ws = [CPWorkspace(world, ql, H, d, device=dev) for _ in range(world)]
    cps = [DirectCPAttention(r, world, ws) for r in range(world)]
    keys = [torch.cat([k[s:e], k[T + r * ql: T + (r + 1) * ql]]) for r, (s, e) in enumerate(bounds)]
    vals = [torch.cat([v[s:e], v[T + r * ql: T + (r + 1) * ql]]) for r, (s, e) in enumerate(bounds)]
    tables = [[local_intervals(iv[o * ql:(o + 1) * ql], s, e, T, own=(o == r), query_start=r * ql) for o in range(world)]
              for r, (s, e) in enumerate(bounds)]
    for r, cp in enumerate(cps):
        cp.publish(q[r * ql:(r + 1) * ql])
    for r, cp in enumerate(cps):
        cp.partials(keys[r], vals[r], tables[r], [ql] * world, scale)
    merged = [cp.merge() for cp in cps]
    for r, (o, l) in enumerate(merged):
        assert torch.allclose(o.float(), out_ref[r * ql:(r + 1) * ql].float(), rtol=2e-2, atol=2e-2)
        assert torch.allclose(l, lse_ref[:, r * ql:(r + 1) * ql], rtol=1e-3, atol=1e-3)
    for r, cp in enumerate(cps):
        cp.publish_grad(dout[r * ql:(r + 1) * ql])
    grads = [cp.grad_partials() for cp in cps]
    tol = dict(rtol=5e-2, atol=3e-2)
    for r, cp in enumerate(cps):
        dq = cp.reduce_grad()
        assert torch.allclose(dq.float(), dq_ref[r * ql:(r + 1) * ql].float(), **tol)
        s, e = bounds[r]
        dk, dv = grads[r]
        assert torch.allclose(dk[: e - s].float(), dk_ref[s:e].float(), **tol)
        assert torch.allclose(dv[: e - s].float(), dv_ref[s:e].float(), **tol)
        assert torch.allclose(dk[e - s:].float(), dk_ref[T + r * ql: T + (r + 1) * ql].float(), **tol)
