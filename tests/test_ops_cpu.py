"""CPU oracles: anchors, interval masks, attention reference and partial merging, losses, optimizer."""
import math

import pytest
import torch

from aspec_b200.ops import anchors as A
from aspec_b200.ops.attention import (build_block_intervals, dense_interval_mask, interval_attention,
                                      interval_attention_reference, merge_partials)
from aspec_b200.ops.vocab_head import head_loss
from aspec_b200.training.lr_scheduler import lr_at_step
from aspec_b200.training.optimizer import BF16Optimizer


def test_anchor_sampling_row_scope():
    T, bs, n_anchor = 64, 4, 8
    lm = torch.zeros(2, T)
    lm[0, 20:] = 1
    lm[1, 60:] = 1          # only 61 is a candidate? 60 (60,61 supervised, <= T-bs=60) -> exactly one
    g = torch.Generator().manual_seed(0)
    anchors, keep = A.sample_anchor_positions(T, lm, n_anchor, bs, generator=g)
    assert anchors.shape == (2, n_anchor) and keep[0].all()
    assert ((anchors[0] >= 20) & (anchors[0] <= T - bs)).all()
    assert keep[1].sum() == 1 and anchors[1][keep[1]].item() == 60 and (anchors[1][~keep[1]] == 0).all()
    # stride: 41 candidates / 8 anchors = 5 -> consecutive (non-wrapped) anchors are 5 apart
    d = (anchors[0][1:] - anchors[0][:-1])
    assert ((d == 5) | (d < 0)).all() and (d < 0).sum() <= 1
    g2 = torch.Generator().manual_seed(0)
    again, _ = A.sample_anchor_positions(T, lm, n_anchor, bs, generator=g2)
    assert torch.equal(again, anchors)
    assert A.anchor_sampling_seed(1, 2, 3, 4) == A.anchor_sampling_seed(1, 2, 3, 4) != A.anchor_sampling_seed(1, 2, 3, 5)


def test_anchor_sampling_document_scope_and_validation():
    lens = (20, 3, 30)
    T = sum(lens)
    docs = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)])[None]
    lm = torch.ones(1, T)
    slots, total, padded = A.document_anchor_slots(lens, 8, 4, alignment=4)
    assert slots == (8, 0, 8) and total == 16 and padded == 16
    anchors, keep = A.sample_document_anchor_positions(lm, docs, lens, 8, 4, generator=torch.Generator().manual_seed(1), alignment=4)
    assert anchors.shape == (1, 16) and keep.all()
    a0, a2 = anchors[0, :8], anchors[0, 8:]
    assert (a0 <= 20 - 4).all() and ((a2 >= 23) & (a2 <= T - 4)).all()
    ok_a, ok_k = A.validate_injected_anchors(anchors, keep, loss_mask=lm, num_anchors=16, block_size=4,
                                             ctx_doc_ids=docs, allow_partial_last_target=True)
    assert torch.equal(ok_a, anchors)
    bad = anchors.clone()
    bad[0, 0] = 18          # block 18..22 crosses into document 1
    with pytest.raises(ValueError):
        A.validate_injected_anchors(bad, keep, loss_mask=lm, num_anchors=16, block_size=4, ctx_doc_ids=docs)
    with pytest.raises(ValueError):
        A.validate_injected_anchors(anchors[:, :5], keep[:, :5], loss_mask=lm, num_anchors=16, block_size=4)


def _visibility_oracle(anchors, keep, T, bs, doc, causal, window):
    n = anchors.numel()
    vis = torch.zeros(n * bs, T + n * bs, dtype=torch.bool)
    for a in range(n):
        if not keep[a]:
            continue
        p = int(anchors[a])
        for j in range(bs):
            for k in range(T):
                ok = k < p and doc[k] == doc[p]
                if window is not None:
                    ok = ok and k >= p - window
                vis[a * bs + j, k] = ok
            for j2 in range(bs):
                vis[a * bs + j, T + a * bs + j2] = (j2 <= j) if causal else True
    return vis


@pytest.mark.parametrize("causal,window", [(False, None), (True, None), (False, 5)])
def test_interval_table_matches_visibility_rule(causal, window):
    T, bs = 40, 3
    doc = torch.tensor([0] * 15 + [1] * 25)
    anchors = torch.tensor([2, 9, 16, 30, 0])
    keep = torch.tensor([True, True, True, True, False])
    start = torch.where(anchors >= 15, 15, 0)
    iv = build_block_intervals(anchors, keep, ctx_len=T, block_size=bs, doc_start=start,
                               context_window=window, causal=causal)
    assert torch.equal(dense_interval_mask(iv, T + 5 * bs), _visibility_oracle(anchors, keep, T, bs, doc, causal, window))


def test_attention_reference_and_partial_merge():
    torch.manual_seed(0)
    T, bs, n = 30, 4, 5
    anchors = torch.tensor([3, 8, 14, 20, 25])
    keep = torch.tensor([True, True, False, True, True])
    iv = build_block_intervals(anchors, keep, ctx_len=T, block_size=bs)
    q = torch.randn(n * bs, 4, 16, dtype=torch.float64)
    k = torch.randn(T + n * bs, 2, 16, dtype=torch.float64)
    v = torch.randn(T + n * bs, 2, 16, dtype=torch.float64)
    out, lse = interval_attention_reference(q, k, v, iv)
    assert (out[2 * bs:3 * bs] == 0).all() and torch.isinf(lse[:, 2 * bs:3 * bs]).all()
    # split the keys in two shards (context halves), attend per shard, merge exactly
    cut = 12
    iv_a = iv.clone(); iv_b = iv.clone()
    iv_a[:, 1] = iv_a[:, 1].clamp(max=cut); iv_a[:, 0] = torch.minimum(iv_a[:, 0], iv_a[:, 1])
    iv_a[:, 2:] = 0
    iv_b[:, 0] = iv_b[:, 0].clamp(min=cut); iv_b[:, 1] = torch.maximum(iv_b[:, 1], iv_b[:, 0])
    oa, la = interval_attention_reference(q, k, v, iv_a)
    ob, lb = interval_attention_reference(q, k, v, iv_b)
    mo, ml = merge_partials(torch.stack([oa, ob]), torch.stack([la, lb]))
    assert torch.allclose(mo, out, atol=1e-10)
    fin = torch.isfinite(lse)
    assert torch.allclose(ml[fin], lse[fin], atol=1e-10) and torch.equal(torch.isfinite(ml), fin)
    # differentiable entry point on CPU == reference
    q32 = q.float().requires_grad_()
    o2, _ = interval_attention(q32, k.float(), v.float(), iv)
    o2.sum().backward()
    assert q32.grad is not None and torch.allclose(o2.double(), out, atol=1e-4)


def test_head_loss_reference_gradients():
    torch.manual_seed(1)
    R, D, V = 12, 8, 50
    h = torch.randn(R, D, requires_grad=True)
    W = torch.randn(V, D)
    labels = torch.randint(0, V, (R,))
    wt = torch.rand(R)
    th = torch.randn(7, D)
    ti = torch.randint(0, 7, (R,), dtype=torch.int32)
    num, ce, l1, correct = head_loss(h, W, labels, wt, teacher_hidden=th, t_index=ti, a_ce=0.3, a_l1=0.7)
    logits = h @ W.t()
    want = (wt * (0.3 * torch.nn.functional.cross_entropy(logits, labels, reduction="none")
                  + 0.7 * (logits.softmax(-1) - (th[ti.long()] @ W.t()).softmax(-1)).abs().sum(-1))).sum()
    assert torch.allclose(num, want, atol=1e-5)
    num.backward()
    assert h.grad.abs().sum() > 0 and (l1 <= 2.0 + 1e-5).all()


def test_lr_schedule_shapes():
    kw = dict(max_lr=1.0, total_steps=100, warmup_steps=10, min_lr=0.1)
    assert lr_at_step(0, **kw) == 0.0 and lr_at_step(5, **kw) == pytest.approx(0.5) and lr_at_step(10, **kw) == 1.0
    assert lr_at_step(55, decay_style="linear", **kw) == pytest.approx(0.55)
    assert lr_at_step(55, decay_style="cosine", **kw) == pytest.approx(0.55)
    assert lr_at_step(100, decay_style="cosine", **kw) == pytest.approx(0.1) and lr_at_step(500, **kw) == 0.1
    assert lr_at_step(50, decay_style="constant", **kw) == 1.0
    assert lr_at_step(40, decay_style="inverse-square-root", **kw) == pytest.approx(0.5)
    w = dict(decay_style="WSD", wsd_decay_steps=20, **kw)
    assert lr_at_step(80, wsd_decay_style="linear", **w) == 1.0
    assert lr_at_step(90, wsd_decay_style="linear", **w) == pytest.approx(0.55)
    assert lr_at_step(90, wsd_decay_style="exponential", **w) == pytest.approx(0.1 + 0.9 * (2 * 0.5 ** 0.5 - 1))
    assert lr_at_step(90, wsd_decay_style="minus_sqrt", **w) == pytest.approx(0.1 + 0.9 * (1 - math.sqrt(0.5)))


def test_flat_optimizer_matches_torch_adamw_and_skips_nonfinite():
    torch.manual_seed(2)
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 3))
    ref = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 3))
    ref.load_state_dict(model.state_dict())
    opt = BF16Optimizer(model, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0, total_steps=100, warmup_ratio=0.0,
                        decay_style="constant")
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.1)
    x = torch.randn(4, 6)
    for _ in range(3):
        model(x).pow(2).sum().backward()
        ref(x).pow(2).sum().backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        norm = opt.step()
        ropt.step(); ropt.zero_grad()
        assert norm > 0
        for a, b in zip(model.parameters(), ref.parameters()):
            assert torch.allclose(a, b, atol=1e-5)
            assert a.grad is None and (a.main_grad == 0).all()
    before = [p.detach().clone() for p in model.parameters()]
    model[0].weight.main_grad[0, 0] = float("nan")
    opt.step()
    for a, b in zip(model.parameters(), before):
        assert torch.equal(a, b)
    assert opt.skipped_steps == 1
    # a skipped update does not advance Adam's bias-correction step: the next applied update is step 4 on both sides
    assert opt.step_count == 3
    model(x).pow(2).sum().backward()
    ref(x).pow(2).sum().backward()
    torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
    opt.step()
    ropt.step(); ropt.zero_grad()
    assert opt.step_count == 4 and opt.skipped_steps == 1
    for a, b in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-5)
    state = opt.state_dict()
    assert state["step"] == 4
    assert set(state["master"]) == {"0.weight", "0.bias", "1.weight", "1.bias"}
    opt.load_state_dict(state)
    assert opt.step_count == 4


def test_sampling_logits_support_and_l1():
    """Temperature / top-k / top-p restrict the support the way a sampler would; default is the identity."""
    import torch
    from aspec_b200.ops.loss_sampling import l1_between, sampling_logits
    torch.manual_seed(0)
    z = torch.randn(5, 50)
    assert sampling_logits(z) is z
    k = sampling_logits(z, (1.0, 1.0, 7))
    assert (torch.isfinite(k).sum(-1) == 7).all()
    assert torch.equal(torch.isfinite(k), z >= z.topk(7, -1).values[:, -1:])
    t = sampling_logits(z, (0.5, 1.0, -1))
    assert torch.allclose(t, (z - z.amax(-1, keepdim=True)) / 0.5)
    p = sampling_logits(z, (1.0, 0.6, -1))
    pr = z.softmax(-1)
    for r in range(5):
        order = pr[r].argsort(descending=True, stable=True)
        before = pr[r][order].cumsum(0) - pr[r][order]
        keep = set(order[before <= 0.6].tolist())
        assert set(torch.isfinite(p[r]).nonzero().flatten().tolist()) == keep
    # identical distributions on identical supports are at distance 0; disjoint supports at distance 2
    assert torch.allclose(l1_between(z, z, (1.0, 0.5, 10), (1.0, 0.5, 10)), torch.zeros(5), atol=1e-6)
    a = torch.full((1, 4), -10.0); a[0, 0] = 10
    b = torch.full((1, 4), -10.0); b[0, 3] = 10
    assert abs(float(l1_between(a, b, (1.0, 1.0, 1), (1.0, 1.0, 1))) - 2.0) < 1e-5


def test_dspark_l1_sampling_changes_the_loss_and_trains():
    import torch
    from aspec_b200.config.draft_config import DSparkConfig
    from aspec_b200.models.draft.dspark import DSparkDraftModel
    from aspec_b200.models.dspark import DSparkModel
    torch.manual_seed(0)
    cfg = DSparkConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=32, vocab_size=128, num_target_layers=2, target_hidden_size=64,
                       target_num_hidden_layers=4, markov_rank=8, mask_token_id=127)
    draft = DSparkDraftModel(cfg)
    head = torch.randn(128, 64) * 0.3
    T = 48
    ids = torch.randint(0, 120, (1, T))
    lm = torch.ones(1, T)
    hs, last = torch.randn(1, T, 128), torch.randn(1, T, 64)
    out = {}
    for name, samp in (("plain", (1.0, 1.0, -1)), ("topk", (0.7, 0.9, 16))):
        model = DSparkModel(draft, block_size=4, num_anchors=8, l1_target_sampling=samp, l1_draft_sampling=samp,
                            deterministic_anchor_sampling=True)
        res = model(ids, hs, lm, head, last_hidden_states=last)
        num = res[6][0]
        draft.zero_grad()
        num.backward()
        g = draft.layers[0].mlp.down_proj.weight.grad
        assert g is not None and torch.isfinite(g).all() and g.abs().sum() > 0
        out[name] = float(res[5]["l1_loss"][0])
    assert out["plain"] != out["topk"]


def test_chunked_head_loss_equals_the_whole_head():
    """Rows in chunks with recomputed logits: same loss, per-row outputs and gradients as one call over all rows."""
    from aspec_b200.ops.vocab_head import head_loss
    torch.manual_seed(0)
    R, D, V, Tt, rk = 37, 16, 64, 20, 4
    W = torch.randn(V, D) * 0.3
    w2 = torch.nn.Parameter(torch.randn(V, rk) * 0.3)
    teacher = torch.randn(Tt, D)
    t_index = torch.randint(0, Tt, (R,), dtype=torch.int32)
    labels = torch.randint(0, V, (R,))
    weight = torch.rand(R)
    outs = []
    for chunk in (0, 8):
        h = torch.randn(R, D, generator=torch.Generator().manual_seed(1)).requires_grad_(True)
        p = torch.randn(R, rk, generator=torch.Generator().manual_seed(2)).requires_grad_(True)
        w2.grad = None
        num, ce, l1, ok = head_loss(h, W, labels, weight, prev_emb=p, markov_w2=w2, teacher_hidden=teacher, t_index=t_index,
                                    a_ce=0.3, a_l1=0.7, chunk_rows=chunk)
        num.backward()
        outs.append((num.detach(), ce, l1, ok, h.grad.clone(), p.grad.clone(), w2.grad.clone()))
    for a, b in zip(*outs):
        assert torch.allclose(a, b, atol=1e-5)
    with torch.no_grad():
        n2, *_ = head_loss(torch.randn(R, D, generator=torch.Generator().manual_seed(1)), W, labels, weight, chunk_rows=8, a_ce=1.0)
        n1, *_ = head_loss(torch.randn(R, D, generator=torch.Generator().manual_seed(1)), W, labels, weight, a_ce=1.0)
    assert torch.allclose(n1, n2, atol=1e-5)
