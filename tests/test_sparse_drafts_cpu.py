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
