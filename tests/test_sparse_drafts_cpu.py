"""Sparse-attention draft variants (DSA / QSA / CSA) and MLA on CPU: with a budget that covers every eligible key
the sparse core must reproduce dense attention, and each training stage must route gradients to the right
parameter set (reference: tests/test_draft_csa.py, tests/test_draft_qsa.py, tests/test_draft_dsa.py)."""
import pytest
import torch

from aspec_b200.config.draft_config import DSparkConfig, K3DSparkConfig
from aspec_b200.models.draft.dspark import DSparkDraftModel
from aspec_b200.models.draft.auto import AutoEagle3DraftModel
from aspec_b200.models.dspark import DSparkModel

BASE = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
            vocab_size=256, num_target_layers=3, target_hidden_size=64, target_num_hidden_layers=8, markov_rank=16,
            mask_token_id=255)
KINDS = {
    "dsa": dict(layer_types=["deepseek_sparse_attention"], dsa_token_budget=64, dsa_index_n_heads=4,
                dsa_index_head_dim=16, dsa_q_lora_rank=16, dsa_rope_dim=8),
    "qsa": dict(layer_types=["qwen_sparse_attention"], qsa_token_budget=64, qsa_compress_ratio=2,
                qsa_index_n_heads=2, qsa_index_head_dim=16, qsa_rope_dim=8),
    "csa": dict(layer_types=["compressed_sparse_attention"], compress_ratios=[4], sliding_window=6, index_topk=64,
                index_n_heads=2, index_head_dim=16),
}


def _run(kind, stage, seed=0):
    torch.manual_seed(seed)
    cfg = DSparkConfig(**BASE, **KINDS[kind], **{f"{kind}_training_stage": stage})
    model = DSparkDraftModel(cfg)
    wrapper = DSparkModel(model, block_size=4, num_anchors=8)
    torch.manual_seed(1)
    ids = torch.randint(0, 250, (1, 48))
    hs, last = torch.randn(1, 48, 192), torch.randn(1, 48, 64)
    mask = torch.ones(1, 48)
    mask[:, :10] = 0
    out = wrapper(ids, hs, mask, torch.randn(256, 64) * 0.1, last_hidden_states=last, anchor_seed=7)
    return model, out


@pytest.mark.parametrize("kind", ["dsa", "qsa", "csa"])
def test_full_budget_sparse_matches_dense(kind):
    dense_model, dense = _run(kind, "dense")
    sparse_model, sparse = _run(kind, "sparse")
    # identical seeds: shared parameters are equal, so the CE terms must agree when nothing is pruned
    d = dict(dense[5])["ce_loss"]
    s = dict(sparse[5])["ce_loss"]
    assert torch.allclose(d[0] / d[1], s[0] / s[1], rtol=2e-4, atol=2e-5)
    assert f"{kind}_indexer_loss" in sparse[5]


@pytest.mark.parametrize("kind", ["dsa", "qsa", "csa"])
def test_stage_gradient_routing(kind):
    for stage, want_indexer, want_main in (("dense", False, True), ("indexer_warmup", True, False), ("sparse", True, True)):
        model, out = _run(kind, stage)
        out[6][0].backward()
        idx = sum(float(p.grad.abs().sum()) for n, p in model.named_parameters() if "indexer" in n and p.grad is not None)
        main = sum(float(p.grad.abs().sum()) for n, p in model.named_parameters()
                   if "indexer" not in n and p.grad is not None)
        assert (idx > 0) == want_indexer, (kind, stage)
        assert (main > 0) == want_main, (kind, stage)
        if stage == "indexer_warmup":
            assert sorted(out[5]) == [f"{kind}_indexer_loss"]


def test_mla_dspark_trains():
    torch.manual_seed(0)
    cfg = K3DSparkConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                         vocab_size=256, num_target_layers=3, target_hidden_size=64, target_num_hidden_layers=8,
                         markov_rank=16, mask_token_id=255, q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16,
                         qk_rope_head_dim=8, v_head_dim=16)
    model = AutoEagle3DraftModel.from_config(cfg)
    assert type(model).__name__ == "K3DSparkModel"
    wrapper = DSparkModel(model, block_size=4, num_anchors=8)
    mask = torch.ones(1, 48)
    out = wrapper(torch.randint(0, 250, (1, 48)), torch.randn(1, 48, 192), mask, torch.randn(256, 64) * 0.1,
                  last_hidden_states=torch.randn(1, 48, 64))
    out[6][0].backward()
    assert model.layers[0].self_attn.kv_b_proj.weight.grad.abs().sum() > 0


def test_dsa_kernel_path_statement_matches_the_chunked_path(monkeypatch):
    """The GPU sparse stage (scores kernel -> top-k kernel -> selected-key kernel, KL on the selected set) is driven
    here through its fp32 statements: loss terms must equal the original chunked formulation."""
    from aspec_b200.ops import sparse_attention as SA
    kind = dict(KINDS["dsa"], dsa_token_budget=6)        # a budget that really prunes
    outs = {}
    for name in ("chunked", "kernel_path"):
        if name == "kernel_path":
            calls = {"n": 0}

            def first_true(q, keys, values):
                calls["n"] += 1
                return calls["n"] == 1           # only the stage dispatch in DSAAttention.forward takes the new path

            monkeypatch.setattr(SA, "_kernel_ok", first_true)
        torch.manual_seed(0)
        cfg = DSparkConfig(**BASE, **kind, dsa_training_stage="sparse")
        model = DSparkDraftModel(cfg)
        wrapper = DSparkModel(model, block_size=4, num_anchors=8)
        torch.manual_seed(1)
        ids = torch.randint(0, 250, (1, 48))
        hs, last = torch.randn(1, 48, 192), torch.randn(1, 48, 64)
        mask = torch.ones(1, 48)
        mask[:, :10] = 0
        out = wrapper(ids, hs, mask, torch.randn(256, 64) * 0.1, last_hidden_states=last, anchor_seed=7)
        out[6][0].backward()
        outs[name] = (dict(out[5]), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None})
    a, b = outs["chunked"], outs["kernel_path"]
    for key in ("ce_loss", "dsa_indexer_loss"):
        assert torch.allclose(a[0][key][0], b[0][key][0], rtol=1e-4, atol=1e-5), key
    assert set(a[1]) == set(b[1])
    for n in a[1]:
        assert torch.allclose(a[1][n], b[1][n], rtol=2e-3, atol=2e-5), n


def test_selected_attention_and_selection_oracles():
    from aspec_b200.ops.attention import interval_attention_reference
    from aspec_b200.ops.sparse_attention import (indexer_scores_reference, selected_attention_reference,
                                                 topk_select_reference)
    torch.manual_seed(3)
    n, hq, hkv, d, T = 6, 4, 2, 16, 30
    q, k, v = torch.randn(n, hq, d), torch.randn(T, hkv, d), torch.randn(T, hkv, d)
    lo = torch.tensor([0, 0, 3, 5, 10, 7])
    hi = torch.tensor([10, 30, 3, 25, 11, 29])
    # a list that names every key of [lo, hi) once (plus empty slots) is interval attention
    sel = torch.full((n, T + 2), -1)
    for i in range(n):
        r = torch.arange(lo[i], hi[i])
        sel[i, 1:1 + r.numel()] = r[torch.randperm(r.numel())]
    out, lse = selected_attention_reference(q, k, v, sel, 0.25)
    iv = torch.stack([lo, hi, torch.zeros_like(lo), torch.zeros_like(lo)], 1)
    want, want_lse = interval_attention_reference(q, k, v, iv, 0.25)
    assert torch.allclose(out, want, atol=1e-5) and torch.allclose(lse[:, [0, 1, 3, 4, 5]], want_lse[:, [0, 1, 3, 4, 5]], atol=1e-5)
    assert (out[2] == 0).all() and torch.isinf(lse[:, 2]).all()
    qi, ki, w = torch.randn(n, 4, 8), torch.randn(T, 8), torch.rand(n, 4)
    sc = indexer_scores_reference(qi, ki, w, lo, hi)
    top = topk_select_reference(sc, lo, hi, 5)
    for i in range(n):
        got = [t for t in top[i].tolist() if t >= 0]
        assert got == sorted(got) and len(got) == min(5, int(hi[i] - lo[i]))
        if got:
            worst = sc[i, got].min()
            rest = [t for t in range(int(lo[i]), int(hi[i])) if t not in got]
            assert all(sc[i, t] <= worst for t in rest)
