"""Guard bands around device allocations (``utils/canary.py``): the checker itself on CPU, and the main kernels run
under it on a GPU with shapes that end inside tiles (where an out-of-bounds store would land in a guard band)."""
import pytest
import torch

from aspec_b200.utils.canary import CanaryError, _Guard, guard_allocations


def test_guard_sees_a_store_past_either_end_and_restores_torch():
    real = torch.empty
    g = _Guard(300)
    v = g.carve((5, 3), torch.float32, "cpu", 0)
    assert v.shape == (5, 3) and float(v.sum()) == 0.0
    g.check()
    raw = g.live[0][0]
    raw[g.pad - 1] = 1
    with pytest.raises(CanaryError, match="before it"):
        g.check()
    raw[g.pad - 1] = 0xA5
    raw[g.pad + 60] = 7
    with pytest.raises(CanaryError, match="after it, first at byte offset 60"):
        g.check()
    with guard_allocations():
        assert torch.zeros(3, 2).shape == (3, 2) and torch.full((2,), 3.0).tolist() == [3.0, 3.0]      # CPU passes through
    assert torch.empty is real


@pytest.mark.gpu
def test_kernels_keep_inside_their_buffers():
    from aspec_b200.ops import attention_sm100 as K
    from aspec_b200.ops import elementwise_sm100 as E
    from aspec_b200.ops import gemm as G
    from aspec_b200.ops.attention import build_block_intervals
    from aspec_b200.ops.gemm import check_status
    from aspec_b200.ops.sparse_attention import indexer_scores, selected_attention_backward, selected_attention_forward, topk_select
    from aspec_b200.ops.vocab_head import head_loss
    dev, bf = "cuda", torch.bfloat16
    torch.manual_seed(0)
    # operands are made outside the block; everything the wrappers allocate inside it is guarded
    a = torch.randn(300, 264, device=dev).to(bf)
    b = torch.randn(520, 264, device=dev).to(bf)
    T, A, bs, H, Hk, d = 700, 40, 4, 4, 2, 128
    anchors = torch.sort(torch.randint(8, T - bs, (A,), device=dev)).values
    q = (torch.randn(A * bs, H, d, device=dev) * 0.5).to(bf)
    k = (torch.randn(T + A * bs, Hk, d, device=dev) * 0.5).to(bf)
    v = (torch.randn(T + A * bs, Hk, d, device=dev) * 0.5).to(bf)
    dout = torch.randn_like(q)
    iv = build_block_intervals(anchors, torch.ones(A, dtype=torch.bool, device=dev), ctx_len=T, block_size=bs)
    sel = torch.sort(torch.randint(0, T, (A * bs, 37), device=dev), dim=1).values.to(torch.int32)
    hidden = torch.randn(150, 128, device=dev).to(bf).requires_grad_()
    lm_w = (torch.randn(1000, 128, device=dev) * 0.2).to(bf)
    labels = torch.randint(0, 1000, (150,), device=dev)
    iq = (torch.randn(200, 8, 128, device=dev) * 0.3).to(bf)
    ik = (torch.randn(900, 128, device=dev) * 0.3).to(bf)
    iw = torch.rand(200, 8, device=dev)
    lo = torch.zeros(200, dtype=torch.int32, device=dev)
    hi = torch.randint(1, 900, (200,), device=dev, dtype=torch.int32)
    x = torch.randn(333, 256, device=dev).to(bf)
    w = torch.rand(256, device=dev).to(bf)
    with guard_allocations() as guard:
        G.gemm(a, b)                                              # 300 x 520 x 264: every dimension ends inside a tile
        G.gemm(a, b, out_dtype=torch.float32)
        o, lse = K.forward(q, k, v, iv, d ** -0.5)
        K.backward(q, k, v, iv, o, lse, dout, d ** -0.5)
        so, sl = selected_attention_forward(q, k, v, sel, d ** -0.5)
        selected_attention_backward(q, k, v, sel, so, sl, dout, d ** -0.5)
        scores = indexer_scores(iq, ik, iw, lo, hi)
        topk_select(scores, lo, hi, 64)
        num, *_ = head_loss(hidden, lm_w, labels, torch.rand(150, device=dev), a_ce=1.0)
        num.backward()
        E.rmsnorm_fwd(x, w, 1e-6)
        torch.cuda.synchronize()
        assert len(guard.live) > 10
    check_status(dev)
