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
    (600, 40, 7, 10, 2, False, None, 1),       # 5 query heads per key head: run as 4 + 1
    (700, 30, 4, 12, 2, True, None, 2),        # 6 per key head: 4 + 2
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
    assert (out.float() - ref.detach()).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        assert err < 6e-2 * max(1.0, b.abs().max().item()), f"{name} err {err}"


def _mla_case(n_ctx, n_blocks, bs, heads, seed, causal=False, docs=1):
    """Materialised-MLA head shape: query / key width 192 (128 + 64 rotary), value width 128, one kv head per head."""
    from aspec_b200.ops.attention import build_block_intervals
    g = torch.Generator(device="cpu").manual_seed(seed)
    doc_len = n_ctx // docs
    anchors = torch.sort(torch.randint(1, n_ctx - bs, (n_blocks,), generator=g)).values
    keep = torch.rand(n_blocks, generator=g) > 0.1
    iv = build_block_intervals(anchors, keep, ctx_len=n_ctx, block_size=bs, doc_start=(anchors // doc_len) * doc_len,
                               causal=causal).cuda()
    Q = n_blocks * bs
    q = (torch.randn(Q, heads, 192, generator=g) * 0.8).cuda().bfloat16()
    k = (torch.randn(n_ctx + Q, heads, 192, generator=g) * 0.8).cuda().bfloat16()
    v = torch.randn(n_ctx + Q, heads, 128, generator=g).cuda().bfloat16()
    return q, k, v, iv


@pytest.mark.parametrize("n_ctx,n_blocks,bs,heads,causal,docs", [
    (200, 9, 7, 2, False, 1),
    (1000, 64, 7, 4, False, 3),
    (2048, 128, 7, 16, True, 2),       # K3 DSpark / DeepSeek EAGLE layout: 16 heads of (192, 128)
])
def test_mla_heads_forward_backward(n_ctx, n_blocks, bs, heads, causal, docs):
    from aspec_b200.ops import attention_sm100 as K
    from aspec_b200.ops.attention import interval_attention, interval_attention_reference
    from aspec_b200.ops.gemm import check_status
    q, k, v, iv = _mla_case(n_ctx, n_blocks, bs, heads, seed=n_ctx + heads, causal=causal, docs=docs)
    assert K.supported(q, k, v)
    scale = 192 ** -0.5
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    out, lse = interval_attention(q, k, v, iv, scale)
    assert out.shape == (q.shape[0], heads, 128)
    do = torch.randn_like(out)
    out.backward(do)
    check_status("cuda")
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref, ref_lse = interval_attention_reference(qr, kr, vr, iv, scale)
    ref.backward(do.float())
    assert (out.float() - ref).abs().max().item() < 3e-2
    fin = torch.isfinite(ref_lse)
    assert torch.equal(fin, torch.isfinite(lse))
    assert (lse[fin] - ref_lse[fin]).abs().max().item() < 2e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        assert a.shape == b.shape
        err = (a.float() - b).abs().max().item()
        assert err < 6e-2 * max(1.0, b.abs().max().item()), f"{name} err {err}"


def test_k3_dspark_and_deepseek_eagle_attention_use_the_kernels():
    """The MLA attention module at the shipped head shape dispatches to the tcgen05 kernels and matches fp32."""
    from types import SimpleNamespace
    from aspec_b200.models.draft.mla import MLAAttention
    from aspec_b200.ops import observed
    from aspec_b200.ops.attention import build_block_intervals
    cfg = SimpleNamespace(hidden_size=256, num_attention_heads=4, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                          kv_lora_rank=64, q_lora_rank=96, rms_norm_eps=1e-6, rope_theta=10000.0)
    torch.manual_seed(0)
    ref = MLAAttention(cfg)
    import copy
    mod = copy.deepcopy(ref).cuda().bfloat16()
    T, nb, bs = 300, 12, 7
    anchors = torch.sort(torch.randint(1, T - bs, (nb,))).values
    iv = build_block_intervals(anchors, torch.ones(nb, dtype=torch.bool), ctx_len=T, block_size=bs)
    x, ctx = torch.randn(nb * bs, 256), torch.randn(T, 256)
    q_pos = (anchors[:, None] + torch.arange(bs)[None]).reshape(-1).to(torch.int32)
    kv_pos = torch.cat([torch.arange(T, dtype=torch.int32), q_pos])
    want = ref(x, ctx, q_pos, kv_pos, iv)
    observed.reset()
    got = mod(x.cuda().bfloat16(), ctx.cuda().bfloat16(), q_pos.cuda(), kv_pos.cuda(), iv.cuda())
    assert "tcgen05_interval_flash" in observed.snapshot().get("attention", {})
    assert (got.float().cpu() - want).abs().max().item() < 5e-2 * max(1.0, want.abs().max().item())
