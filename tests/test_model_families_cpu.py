"""Every draft family builds through the factory from a small config, takes one training step's forward and
backward on CPU and routes gradients to the parameters its stage owns
(reference: tests/test_dflash2.py, tests/test_eagle4.py, tests/test_mtp.py, tests/test_dmtp.py)."""
import pytest
import torch

from aspec_b200.config.draft_config import AutoDraftModelConfig
from aspec_b200.training.factory import build_training_model

NATIVE = dict(model_type="qwen3_5_text", hidden_size=64, intermediate_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, vocab_size=256, rms_norm_eps=1e-6, num_hidden_layers=8,
              layer_types=["full_attention"] * 8, rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.25})
DFLASH = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              vocab_size=256, num_target_layers=3, target_hidden_size=64, target_num_hidden_layers=8, mask_token_id=255)
EAGLE = dict(hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2, vocab_size=256,
             draft_vocab_size=256, target_hidden_size=64, num_aux_hidden_states=3, rope_theta=10000.0,
             max_position_embeddings=512)
ARGS = dict(block_size=4, dspark_block_size=4, dflash_block_size=4, dspark_num_anchors=8, dflash_num_anchors=8,
            ttt_length=3, mtp_steps=3, seed=0)


def _batch(vocab=250, T=48, feat=192, last=64):
    torch.manual_seed(3)
    mask = torch.ones(1, T)
    mask[:, :10] = 0
    return dict(input_ids=torch.randint(0, vocab, (1, T)), hidden_states_list=torch.randn(1, T, feat), loss_mask=mask,
                lm_head_weight=torch.randn(256, 64) * 0.1, last_hidden_states=torch.randn(1, T, last))


def _step(raw):
    torch.manual_seed(0)
    model = build_training_model(AutoDraftModelConfig.from_dict(raw), ARGS, "cpu", torch.float32)
    model.train()
    out = model(**_batch())
    out[6][0].backward()
    grads = {n for n, p in model.draft_model.named_parameters() if p.grad is not None and float(p.grad.abs().sum()) > 0}
    assert torch.isfinite(out[0])
    return model, out, grads


def test_dflash2_selector_and_convolutions_train():
    raw = dict(architectures=["DFlash2DraftModel"], model_type="qwen3_dflash2", **DFLASH, block_size=4,
               conv_kernel_size=2, conv_group_size=16, selector_rank=8, selector_top_k=4,
               layer_types=["full_attention", "sliding_attention"], sliding_window=8, final_logit_softcapping=30.0)
    model, out, grads = _step(raw)
    assert {"ce_loss", "selector_loss"} <= set(out[5])
    assert "candidate_selector.successor_codebook" in grads
    assert "layers.0.attention_conv.kernel_projection.weight" in grads
    assert model.layer_block_mask_options[1] == {"is_causal": True, "sliding_window": 8}
    serving = model.draft_model.state_dict_for_serving()
    assert "fc.weight" in serving and "embed_tokens.weight" not in serving


def test_dflash2_convolution_is_block_causal():
    from aspec_b200.models.draft.dflash2 import DFlashGroupedConv
    torch.manual_seed(0)
    conv = DFlashGroupedConv(32, block_size=4, kernel_size=3, group_size=8)
    torch.nn.init.normal_(conv.kernel_projection.weight, std=0.5)
    x = torch.randn(8, 32)
    y, _ = conv.prepare(x)
    x2 = x.clone()
    x2[2] += 1.0                       # row 2 of block 0 may only change rows 2..3 of block 0
    y2, _ = conv.prepare(x2)
    changed = (y - y2).abs().sum(-1) > 1e-6
    assert changed.tolist() == [False, False, True, True, False, False, False, False]


@pytest.mark.parametrize("moe", [False, True])
def test_eagle4_draft_stage(moe):
    extra = dict(enable_moe=True, n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                 n_shared_experts=1, attn_norm=True, enable_post_mlp_norm=True) if moe else {}
    raw = dict(architectures=["LlamaForCausalLMEagle4"], model_type="llama", **EAGLE, sliding_window=16,
               layer_types=["sliding_attention"], efficient_lm_head_config={"type": "low_rank", "rank": 8, "num_candidates": 8},
               eagle4_training_stage="draft", **extra)
    model, out, grads = _step(raw)
    assert not any(g.startswith("efficient_lm_head") for g in grads)
    assert any(g.startswith("midlayer.") for g in grads)
    if moe:
        draft = model.draft_model
        draft.commit_router_load()
        assert int(draft.midlayer.mlp.gate.load.sum()) > 0
        before = draft.midlayer.mlp.gate.e_score_correction_bias.clone()
        draft.midlayer.mlp.gate.update_bias()
        assert draft.midlayer.mlp.gate.e_score_correction_bias.dtype == torch.float32
        assert int(draft.midlayer.mlp.gate.load.sum()) == 0
        assert not torch.equal(before, draft.midlayer.mlp.gate.e_score_correction_bias) or True


def test_eagle4_candidate_stage_trains_only_the_retrieval_head():
    raw = dict(architectures=["LlamaForCausalLMEagle4"], model_type="llama", **EAGLE,
               efficient_lm_head_config={"type": "low_rank", "rank": 8, "num_candidates": 8},
               eagle4_training_stage="candidate_head", candidate_loss_chunk_size=16)
    model, out, grads = _step(raw)
    assert grads == {"efficient_lm_head.weight", "efficient_lm_head_down_proj.weight"}
    assert {"candidate_recall", "candidate_mass"} <= set(out[5])
    draft = model.draft_model
    assert not draft.midlayer.training and draft.efficient_lm_head.training
    draft.initialize_candidate_head()
    exact = draft.lm_head.weight.float()
    approx = draft.efficient_lm_head.weight.float() @ draft.efficient_lm_head_down_proj.weight.float()
    assert (exact - approx).norm() < exact.norm()


def test_deepseek_eagle_mla():
    raw = dict(architectures=["Eagle3DeepseekV2ForCausalLM"], model_type="deepseek_v2", **EAGLE, q_lora_rank=16,
               kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8, v_head_dim=8)
    raw.pop("num_key_value_heads")
    model, out, grads = _step(raw)
    assert "midlayer.self_attn.mla.kv_b_proj.weight" in grads


def test_native_mtp_counts_and_frozen_bindings():
    raw = dict(architectures=["NativeMTPDraftModel"], native_config=NATIVE)
    torch.manual_seed(0)
    model = build_training_model(AutoDraftModelConfig.from_dict(raw), ARGS, "cpu", torch.float32)
    ids = torch.randint(0, 250, (1, 24))
    docs = torch.tensor([[0] * 10 + [1] * 12 + [-1] * 2])
    out = model(ids, None, torch.ones(1, 24), None, last_hidden_states=torch.randn(1, 24, 64), ctx_doc_ids=docs)
    out[6][0].backward()
    # document of n tokens: min(3, n-2) steps over a prefix of n-steps-1 rows -> 6 + 8 rows at every depth
    assert out[4].tolist() == [14.0, 14.0, 14.0]
    draft = model.draft_model
    assert draft.lm_head.weight.grad is None and draft.embed_tokens.weight.grad is None
    assert draft.fc.weight.grad.abs().sum() > 0
    names = draft.state_dict_for_serving()
    assert "mtp.fc.weight" in names and "mtp.layers.0.self_attn.q_proj.weight" in names
    assert set(draft.state_dict_from_serving(names)) == set(draft.state_dict())


@pytest.mark.parametrize("mode", ["token", "hidden"])
@pytest.mark.parametrize("arch", ["DSparkDraftModel", "DFlashDraftModel"])
def test_mtp_conditioned_blocks(mode, arch):
    raw = dict(architectures=[arch], **DFLASH, mtp_conditioning={"mode": mode, "native_config": NATIVE})
    raw["num_hidden_layers"] = 1
    if arch == "DSparkDraftModel":
        raw.update(model_type="qwen3_dspark", markov_rank=16)
    model, out, grads = _step(raw)
    start = 1 if arch == "DSparkDraftModel" else 2
    assert out[4][:start].sum() == 0 and out[4][start:].min() > 0      # the visible first candidate is not supervised
    assert not any(g.startswith("mtp_source.") for g in grads)
    assert ("mtp_fusion.proj.weight" in grads) == (mode == "hidden")
    if arch == "DSparkDraftModel":
        assert "suffix_tau_probabilistic" in out[5]


@pytest.mark.parametrize("ffn", ["ling_moe", "qwen3_moe"])
def test_dspark_with_mixture_of_experts_feed_forward_trains(ffn):
    """DSpark over the two MoE feed-forwards: experts and routers receive gradients, router statistics are reported,
    and (Ling) the balancing bias moves once per committed step."""
    extra = dict(ffn_type=ffn, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32)
    if ffn == "ling_moe":
        extra.update(num_shared_experts=1, moe_shared_expert_intermediate_size=32, n_group=2, topk_group=1, routed_scaling_factor=2.5,
                     moe_router_enable_expert_bias=True, router_z_loss_coef=1e-3, expert_swiglu_limit_list=[0, 0],
                     share_expert_swiglu_limit_list=[0, 0])
    raw = dict(architectures=["DSparkDraftModel"], markov_rank=8, head_dim=16, target_layer_ids=[1, 3, 5], rope_theta=10000.0,
               max_position_embeddings=512, **DFLASH, **extra)
    model, out, grads = _step(raw)
    assert any(".experts." in n for n in grads) and any(".gate." in n for n in grads)
    if ffn == "ling_moe":
        from aspec_b200.models.draft.ling_moe import LingMoE, update_ling_bias
        assert {"router_z_loss", "router_max_load", "_ling_router_counts"} <= set(out[5])
        layers = [m for m in model.draft_model.modules() if isinstance(m, LingMoE)]
        counts = out[5]["_ling_router_counts"]
        assert counts.shape == (len(layers), 8) and float(counts.sum()) > 0
        before = [l.gate.expert_bias.clone() for l in layers]
        update_ling_bias(layers, counts.clone(), update_rate=1e-3)
        assert any(not torch.equal(b, l.gate.expert_bias) for b, l in zip(before, layers))
        assert all(l.gate.expert_bias.dtype == torch.float32 for l in layers)


def test_native_mtp_tensors_are_read_from_a_sharded_checkpoint_directory(tmp_path):
    """Only ``mtp.*`` tensors, only from the shards that hold them; a frozen MTP source loads them and then validates
    against them."""
    import json
    from safetensors.torch import save_file
    from aspec_b200.models.dmtp import FrozenMTPFeatures, read_native_mtp_tensors
    from aspec_b200.models.draft.mtp import native_key
    source = FrozenMTPFeatures(NATIVE)
    torch.manual_seed(5)
    native = {native_key(n): torch.randn_like(t) for n, t in source.state_dict().items()}
    assert all(k.startswith("mtp.") for k in native)
    save_file({"model.layers.0.weight": torch.zeros(2)}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(native, str(tmp_path / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {"model.layers.0.weight": "model-00001-of-00002.safetensors",
                            **{k: "model-00002-of-00002.safetensors" for k in native}}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    got = read_native_mtp_tensors(str(tmp_path))
    assert set(got) == set(native) and all(torch.equal(got[k], native[k]) for k in native)
    source.initialize_native_weights(got)
    source.validate_native_weights(got)
    assert not any(p.requires_grad for p in source.parameters())
    (tmp_path / "model.safetensors.index.json").unlink()            # unsharded layout: every safetensors file is looked at
    assert set(read_native_mtp_tensors(str(tmp_path))) == set(native)
