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


def test_rope_llama3_dynamic_and_multi_axis_families():
    import math
    import torch
    from aspec_b200.config.rope import mrope_axis_of_frequency
    from aspec_b200.ops.rope import qk_norm_rope, qk_norm_rope_reference
    d, theta = 128, 5e5
    base, _ = rope_inverse_frequencies(d, {"rope_theta": theta, "rope_type": "default"})
    p = {"rope_theta": theta, "rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
         "original_max_position_embeddings": 8192}
    got, att = rope_inverse_frequencies(d, p)
    assert att == 1.0
    for f, g in zip(base, got):
        wave = 2 * math.pi / f
        if wave < 8192 / 4.0:
            assert g == f
        elif wave > 8192 / 1.0:
            assert g == pytest.approx(f / 8.0)
        else:
            assert f / 8.0 <= g <= f
    assert got[0] == base[0] and got[-1] == pytest.approx(base[-1] / 8.0)
    try:                                         # the same rule as stated by the transformers library, where it is importable
        from transformers import LlamaConfig
        from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
        hf = LlamaConfig(hidden_size=d * 4, num_attention_heads=4, max_position_embeddings=131072,
                         rope_parameters=dict(p, rope_type="llama3"))
        want, _ = ROPE_INIT_FUNCTIONS["llama3"](hf, "cpu")
        assert torch.allclose(torch.tensor(got), want.float(), rtol=1e-5)
    except (ImportError, TypeError, KeyError, AttributeError):
        pass
    # dynamic NTK: unchanged inside the trained window, a larger base beyond it
    dyn = {"rope_theta": 1e4, "rope_type": "dynamic", "factor": 2.0, "original_max_position_embeddings": 2048}
    same, _ = rope_inverse_frequencies(64, dict(dyn, sequence_length=2048))
    plain, _ = rope_inverse_frequencies(64, {"rope_theta": 1e4, "rope_type": "default"})
    assert same == plain
    longer, _ = rope_inverse_frequencies(64, dict(dyn, sequence_length=8192))
    grown = 1e4 * ((2.0 * 8192 / 2048) - 1.0) ** (64 / 62)
    assert longer[1] == pytest.approx(grown ** (-2 / 64)) and longer[-1] < plain[-1]
    with pytest.raises(ValueError):
        rope_inverse_frequencies(64, {"rope_theta": 1e4, "rope_type": "longrope", "factor": 2.0})
    # multi-axis: equal streams are ordinary RoPE; distinct streams rotate each frequency band by its own stream
    axes = mrope_axis_of_frequency(16, [2, 3, 3])
    assert axes == [0, 0, 1, 1, 1, 2, 2, 2]
    with pytest.raises(ValueError):
        mrope_axis_of_frequency(16, [2, 3])
    x = torch.randn(5, 2, 16)
    inv = torch.tensor(rope_inverse_frequencies(16, {"rope_theta": 1e4, "rope_type": "mrope"})[0])
    pos = torch.arange(5)
    a = qk_norm_rope(x, None, torch.stack([pos, pos, pos]), inv, 0.0, 1.0, torch.tensor(axes))
    assert torch.equal(a, qk_norm_rope_reference(x, None, pos, inv, 0.0))
    streams = torch.stack([pos, pos + 3, pos * 2])
    b = qk_norm_rope(x, None, streams, inv, 0.0, 1.0, torch.tensor(axes))
    for band, axis in ((slice(0, 2), 0), (slice(2, 5), 1), (slice(5, 8), 2)):
        one = qk_norm_rope_reference(x, None, streams[axis], inv, 0.0)
        assert torch.allclose(b[..., band], one[..., band]) and torch.allclose(b[..., 8:][..., band], one[..., 8:][..., band])
