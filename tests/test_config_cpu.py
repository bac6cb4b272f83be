"""Draft config policies: parsing, defaults and fail-closed validation."""
import json

import pytest

from aspec_b200.config.draft_attention import (context_shard_alignment, resolve_attention_policy,
                                               resolve_head_layout, thd_contract)
from aspec_b200.config.draft_config import (AutoDraftModelConfig, DSparkConfig, draft_model_semantics,
                                            resolve_draft_algorithm)
from aspec_b200.config.draft_structure import resolve_ffn_policy
from aspec_b200.config.rope import resolve_rope_theta, rope_inverse_frequencies


def test_head_layouts():
    assert resolve_head_layout({"hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8})["type"] == "gqa"
    assert resolve_head_layout({"hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 4})["type"] == "mha"
    assert resolve_head_layout({"hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 1})["type"] == "mqa"
    mla = resolve_head_layout({"model_type": "k3_dspark", "num_attention_heads": 16, "num_key_value_heads": 16})
    assert mla["type"] == "mla_materialized" and mla["head_dim"] == 192
    with pytest.raises(ValueError):
        resolve_head_layout({"num_attention_heads": 6, "num_key_value_heads": 4})
    with pytest.raises(ValueError):
        resolve_head_layout({"hidden_size": 100, "num_attention_heads": 3, "num_key_value_heads": 3})


def test_attention_schedule_and_windows():
    p = resolve_attention_policy({"num_hidden_layers": 2, "sliding_window": 1024})
    assert p["layer_types"] == ["sliding_attention"] * 2 and p["context_windows"] == [1024, 1024]
    assert p["window_semantics"] == "anchor_context"
    p = resolve_attention_policy({"num_hidden_layers": 2, "architectures": ["DFlash2DraftModel"],
                                  "sliding_window": 64, "layer_types": ["full_attention", "sliding_attention"]})
    assert p["window_semantics"] == "query_relative" and p["draft_block_attention"] == ["bidirectional", "causal"]
    with pytest.raises(ValueError):
        resolve_attention_policy({"num_hidden_layers": 1, "layer_types": ["sliding_attention"]})
    with pytest.raises(ValueError):
        resolve_attention_policy({"num_hidden_layers": 2, "layer_types": ["qwen_sparse_attention", "deepseek_sparse_attention"]})
    with pytest.raises(ValueError):
        resolve_attention_policy({"num_hidden_layers": 1, "dsa_token_budget": 64})


def test_sparse_policies_and_alignment():
    dsa = resolve_attention_policy({"num_hidden_layers": 1, "layer_types": ["deepseek_sparse_attention"],
                                    "dsa_training_stage": "sparse", "dsa_index_n_heads": 64, "dsa_token_budget": 2048})
    assert dsa["dsa"]["index_n_heads"] == 64 and dsa["dsa"]["indexer_input_detached"]
    assert thd_contract(dsa)["kernel_mode"] == "varlen_selected"
    qsa = resolve_attention_policy({"num_hidden_layers": 1, "layer_types": ["qwen_sparse_attention"],
                                    "qsa_compress_ratio": 8, "qsa_token_budget": 1024})
    assert qsa["qsa"]["block_topk"] == 128 and context_shard_alignment(qsa) == 8
    csa = resolve_attention_policy({"num_hidden_layers": 2, "sliding_window": 128, "compress_ratios": [4, 0]})
    assert csa["layer_types"] == ["compressed_sparse_attention", "sliding_attention"]
    assert context_shard_alignment(csa) == 4
    with pytest.raises(ValueError):
        resolve_attention_policy({"num_hidden_layers": 1, "layer_types": ["qwen_sparse_attention"],
                                  "qsa_token_budget": 1001})
    with pytest.raises(ValueError):
        resolve_attention_policy({"num_hidden_layers": 1, "layer_types": ["deepseek_sparse_attention"],
                                  "dsa_training_stage": "indexer_warmup", "dsa_indexer_loss_coef": 0})


def test_ffn_policies():
    assert resolve_ffn_policy({}) == {"ffn_type": "dense"}
    q = resolve_ffn_policy({"ffn_type": "qwen3_moe", "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64})
    assert q["router_aux_loss_coef"] == 0.001
    ling = resolve_ffn_policy({"ffn_type": "ling_moe", "num_experts": 64, "num_experts_per_tok": 8,
                               "moe_intermediate_size": 64, "n_group": 8, "topk_group": 4,
                               "moe_shared_expert_intermediate_size": 64, "num_hidden_layers": 1})
    assert ling["routed_scaling_factor"] == 2.5 and ling["router_z_loss_coef"] == pytest.approx(3.5e-6)
    with pytest.raises(ValueError):
        resolve_ffn_policy({"num_experts": 4})
    with pytest.raises(ValueError):
        resolve_ffn_policy({"ffn_type": "qwen3_moe", "num_experts": 4, "num_experts_per_tok": 8, "moe_intermediate_size": 8})
    with pytest.raises(ValueError):
        resolve_ffn_policy({"ffn_type": "ling_moe", "num_experts": 8, "num_experts_per_tok": 8, "moe_intermediate_size": 8,
                            "n_group": 8, "moe_shared_expert_intermediate_size": 8, "num_hidden_layers": 1})


def test_rope():
    assert resolve_rope_theta({"rope_parameters": {"rope_theta": 5e5}}) == 5e5
    with pytest.raises(ValueError):
        resolve_rope_theta({"rope_theta": 1e4, "rope_parameters": {"rope_theta": 1e6}})
    inv, att = rope_inverse_frequencies(8, {"rope_theta": 10000.0, "rope_type": "default"})
    assert len(inv) == 4 and inv[0] == 1.0 and att == 1.0
    inv_l, _ = rope_inverse_frequencies(8, {"rope_theta": 10000.0, "rope_type": "linear", "factor": 4.0})
    assert inv_l[1] == pytest.approx(inv[1] / 4)
    inv_y, att_y = rope_inverse_frequencies(128, {"rope_theta": 1e6, "rope_type": "yarn", "factor": 8.0,
                                                  "original_max_position_embeddings": 32768})
    assert inv_y[0] == pytest.approx(1.0) and inv_y[-1] < inv_y[0] and att_y > 1.0


def test_auto_config_roundtrip(tmp_path):
    cfg = DSparkConfig(hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2,
                       vocab_size=256, num_target_layers=3, target_hidden_size=64, markov_rank=16)
    assert resolve_draft_algorithm(cfg.to_dict()) == "dspark"
    cfg.save_pretrained(str(tmp_path))
    back = AutoDraftModelConfig.from_file(str(tmp_path / "config.json"))
    assert isinstance(back, DSparkConfig) and back.to_dict() == cfg.to_dict()
    sem = draft_model_semantics(cfg)
    assert sem["markov_rank"] == 16 and sem["head_dim"] == 16
    with pytest.raises(ValueError):
        AutoDraftModelConfig.from_dict({"architectures": ["Nope"]})
    with pytest.raises(ValueError):
        DSparkConfig(markov_rank=0, enable_confidence_head=True)
    json.dumps(cfg.to_dict())
