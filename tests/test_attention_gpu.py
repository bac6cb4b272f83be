"""Interval flash attention (tcgen05) against the fp32 dense-mask reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(n_ctx, n_blocks, bs, hq, hkv, seed, causal=False, window=None, docs=1):
    from aspec_b200.ops.attention import build_block_intervals
    g = torch.Generator(device="cpu").manual_seed(seed)
    d = 128
    doc_len = n_ctx // docs
    anchors = torch.sort(torch.randint(1, n_ctx - bs, (n_blocks,), generator=g)).values
    keep = torch.rand(n_blocks, generator=g) > 0.1
    doc_start = (anchors // doc_len) * doc_len
    iv = build_block_intervals(anchors, keep, ctx_len=n_ctx, block_size=bs, doc_start=doc_start,
                               context_window=window, causal=causal).cuda()
    Q = n_blocks * bs
    q = torch.randn(Q, hq, d, generator=g).cuda().bfloat16()
    k = torch.randn(n_ctx + Q, hkv, d, generator=g).cuda().bfloat16()
    v = torch.randn(n_ctx + Q, hkv, d, generator=g).cuda().bfloat16()
    return q, k, v, iv


@pytest.mark.parametrize("n_ctx,n_blocks,bs,hq,hkv,causal,window,docs", [
    (200, 9, 7, 4, 1, False, None, 1),
    (1000, 64, 7, 8, 2, False, None, 3),
    (517, 33, 4, 2, 2, True, None, 1),
    (2048, 128, 7, 8, 2, False, 300, 2),
    (300, 20, 16, 16, 1, False, None, 1),
])
def test_forward_matches_reference(n_ctx, n_blocks, bs, hq, hkv, causal, window, docs):
    from aspec_b200.ops import attention_sm100 as K
    from aspec_b200.ops.attention import interval_attention_reference
    from aspec_b200.ops.gemm import check_status
    q, k, v, iv = _case(n_ctx, n_blocks, bs, hq, hkv, seed=n_ctx, causal=causal, window=window, docs=docs)
    scale = 128 ** -0.5
    out, lse = K.forward(q, k, v, iv, scale)
    check_status("cuda")
    ref, ref_lse = interval_attention_reference(q.float(), k.float(), v.float(), iv, scale)
    assert (out.float() - ref).abs().max().item() < 3e-2
    fin = torch.isfinite(ref_lse)
    assert torch.equal(fin, torch.isfinite(lse))
    assert (lse[fin] - ref_lse[fin]).abs().max().item() < 2e-2


@pytest.mark.parametrize("n_ctx,n_blocks,bs,hq,hkv,causal,window,docs", [
    (200, 9, 7, 4, 1, False, None, 1),
    (1000, 64, 7, 8, 2, False, None, 1),
    (517, 33, 4, 2, 2, True, None, 1),
    (2048, 128, 7, 8, 2, False, 300, 1),       # context window
    (1536, 96, 7, 8, 2, False, None, 3),       # several packed documents
    (1500, 90, 7, 8, 2, True, 256, 3),         # window + causal inside the block + documents
    (4096, 512, 7, 32, 8, False, None, 1),     # the production head layout: 32 / 8 heads, 4 K context, 3584 queries
])
def test_backward_matches_reference(n_ctx, n_blocks, bs, hq, hkv, causal, window, docs):
    from aspec_b200.ops.attention import interval_attention, interval_attention_reference
    from aspec_b200.ops.gemm import check_status
    q, k, v, iv = _case(n_ctx, n_blocks, bs, hq, hkv, seed=7 + n_ctx, causal=causal, window=window, docs=docs)
    scale = 128 ** -0.5
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    out, _ = interval_attention(q, k, v, iv, scale)
    do = torch.randn_like(out)
    out.backward(do)
    check_status("cuda")
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref, _ = interval_attention_reference(qr, kr, vr, iv, scale)
    ref.backward(do.float())
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        assert err < 6e-2 * max(1.0, b.abs().max().item()), f"{name} err {err}"
