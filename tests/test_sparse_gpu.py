"""Sparse-attention kernels (selected-key attention forward / backward, lightning-indexer scores, radix top-k) against
their fp32 PyTorch statements, on small and odd shapes: partial last tiles, empty slots inside lists, empty lists,
duplicate selections of one key by many queries, rows with fewer eligible keys than the budget."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lists(n, T, L, seed, empty_rows=(), hole_rate=0.15):
    g = torch.Generator().manual_seed(seed)
    sel = torch.stack([torch.randperm(T, generator=g)[:L] if L <= T else torch.randint(0, T, (L,), generator=g)
                       for _ in range(n)])
    holes = torch.rand(n, L, generator=g) < hole_rate
    sel = torch.where(holes, torch.full_like(sel, -1), sel)
    for r in empty_rows:
        sel[r] = -1
    return sel.to(torch.int32)


@pytest.mark.parametrize("n,T,L,hq,hkv", [
    (5, 300, 100, 4, 1),        # one partial tile
    (37, 500, 300, 8, 2),       # three tiles, last partial, G = 4
    (9, 2100, 2055, 32, 8),     # the DSA layout: 2048 selected + 7 own-block keys, 32 / 8 heads
    (3, 64, 130, 16, 1),        # G = 16, list longer than the key array (duplicates)
    (4, 200, 128, 2, 2),        # G = 1, exactly one full tile
])
def test_selected_attention_forward_backward(n, T, L, hq, hkv):
    from aspec_b200.ops.gemm import check_status
    from aspec_b200.ops.sparse_attention import selected_attention, selected_attention_reference
    torch.manual_seed(n * 1000 + L)
    q = torch.randn(n, hq, 128).cuda().bfloat16().requires_grad_()
    k = torch.randn(T, hkv, 128).cuda().bfloat16().requires_grad_()
    v = torch.randn(T, hkv, 128).cuda().bfloat16().requires_grad_()
    sel = _lists(n, T, L, seed=L, empty_rows=(1,) if n > 2 else ()).cuda()
    scale = 128 ** -0.5
    out, lse = selected_attention(q, k, v, sel, scale)
    do = torch.randn_like(out)
    out.backward(do)
    check_status("cuda")
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref, ref_lse = selected_attention_reference(qr, kr, vr, sel, scale)
    ref.backward(do.float())
    assert (out.float() - ref).abs().max().item() < 3e-2
    fin = torch.isfinite(ref_lse)
    assert torch.equal(fin, torch.isfinite(lse))
    assert (lse[fin] - ref_lse[fin]).abs().max().item() < 2e-2
    if n > 2:
        assert (out[1] == 0).all()
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        assert err < 6e-2 * max(1.0, b.abs().max().item()), f"{name} err {err}"


@pytest.mark.parametrize("n,T,H,d", [(20, 1000, 64, 128), (7, 333, 8, 64), (130, 4100, 16, 128), (3, 100, 128, 64)])
def test_indexer_scores(n, T, H, d):
    from aspec_b200.ops.gemm import check_status
    from aspec_b200.ops.sparse_attention import indexer_scores, indexer_scores_reference
    torch.manual_seed(n + T)
    qi = torch.randn(n, H, d).cuda().bfloat16()
    ki = torch.randn(T, d).cuda().bfloat16()
    w = torch.rand(n, H).cuda() * 0.1
    lo = torch.randint(0, T // 2, (n,)).cuda()
    hi = (lo + torch.randint(0, T // 2 + 1, (n,)).cuda()).clamp(max=T)
    hi[0] = lo[0]                                          # a row with nothing eligible
    got = indexer_scores(qi, ki, w, lo, hi)
    check_status("cuda")
    want = indexer_scores_reference(qi.float(), ki.float(), w, lo, hi)
    fin = torch.isfinite(want)
    assert torch.equal(fin, torch.isfinite(got))
    assert (got[fin] - want[fin]).abs().max().item() < 2e-2 * max(1.0, want[fin].abs().max().item())


@pytest.mark.parametrize("n,T,k", [(16, 5000, 64), (5, 70000, 2048), (8, 300, 512), (3, 1000, 1)])
def test_topk_select(n, T, k):
    from aspec_b200.ops.sparse_attention import topk_select
    torch.manual_seed(T + k)
    scores = torch.randn(n, T).cuda()
    lo = torch.randint(0, T // 3, (n,)).cuda()
    hi = (lo + torch.randint(1, T - T // 3, (n,)).cuda()).clamp(max=T)
    hi[0] = lo[0] + min(k // 2 + 1, T - int(lo[0]))        # fewer eligible keys than the budget
    if n > 2:
        hi[2] = lo[2]                                      # nothing eligible
    # heavy ties: quantised scores in one row
    scores[1] = (scores[1] * 2).round() / 2
    got = topk_select(scores, lo, hi, k).cpu()
    sc, lo_c, hi_c = scores.cpu(), lo.cpu(), hi.cpu()
    for r in range(n):
        idx = [t for t in got[r].tolist() if t >= 0]
        cnt = int(hi_c[r] - lo_c[r])
        assert len(idx) == min(k, cnt) and idx == sorted(idx) and len(set(idx)) == len(idx)
        assert all(lo_c[r] <= t < hi_c[r] for t in idx)
        assert all(t == -1 for t in got[r, len(idx):].tolist())
        if idx and cnt > k:
            picked = sc[r, idx]
            rest = torch.ones(T, dtype=torch.bool)
            rest[idx] = False
            rest[: lo_c[r]] = False
            rest[hi_c[r]:] = False
            assert picked.min() >= sc[r][rest].max()


def test_dsa_sparse_stage_runs_on_the_kernels():
    """A DSpark draft with a DSA layer in the sparse stage: forward + backward through the kernels, loss finite, the
    dispatchers report the kernels, and the result agrees with the fp32 CPU model within bf16 tolerance."""
    from aspec_b200.config.draft_config import DSparkConfig
    from aspec_b200.models.draft.dspark import DSparkDraftModel
    from aspec_b200.models.dspark import DSparkModel
    from aspec_b200.ops import observed
    from aspec_b200.ops.gemm import check_status
    cfg = DSparkConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=4,
                       num_key_value_heads=1, head_dim=128, vocab_size=2048, num_target_layers=3, target_hidden_size=256,
                       target_num_hidden_layers=8, markov_rank=32, mask_token_id=2047,
                       layer_types=["deepseek_sparse_attention"], dsa_token_budget=48, dsa_index_n_heads=8,
                       dsa_index_head_dim=64, dsa_q_lora_rank=64, dsa_rope_dim=32, dsa_training_stage="sparse")
    torch.manual_seed(0)
    draft = DSparkDraftModel(cfg)
    T = 400
    ids = torch.randint(0, 2000, (1, T))
    hs, last = torch.randn(1, T, 768), torch.randn(1, T, 256)
    mask = torch.cat([torch.zeros(1, 60), torch.ones(1, T - 60)], 1)
    head = torch.randn(2048, 256) * 0.05
    from aspec_b200.ops.anchors import sample_anchor_positions
    anchors, keep = sample_anchor_positions(T, mask, 24, 7, generator=torch.Generator().manual_seed(11))
    ref_model = DSparkModel(draft, block_size=7, num_anchors=24)
    ref = ref_model(ids, hs, mask, head, last_hidden_states=last, injected_anchors=anchors, injected_keep_mask=keep)
    import copy
    gpu_draft = copy.deepcopy(draft).cuda().bfloat16()
    gpu_model = DSparkModel(gpu_draft, block_size=7, num_anchors=24)
    observed.reset()
    out = gpu_model(ids.cuda(), hs.cuda().bfloat16(), mask.cuda(), head.cuda().bfloat16(),
                    last_hidden_states=last.cuda().bfloat16(), injected_anchors=anchors, injected_keep_mask=keep)
    out[6][0].backward()
    check_status("cuda")
    seen = observed.snapshot()
    assert "tcgen05_selected_keys" in seen.get("sparse_attention", {})
    assert "tcgen05_relu_weighted_head_sum" in seen.get("indexer", {})
    assert "radix_select" in seen.get("topk", {})
    assert torch.isfinite(out[0])
    assert abs(float(out[0]) - float(ref[0])) < 0.15 * max(1.0, abs(float(ref[0])))
    g = gpu_draft.layers[0].self_attn.indexer.q_b_proj.weight
    assert (g.grad is not None and torch.isfinite(g.grad.float()).all()) or getattr(g, "main_grad", None) is not None
