"""Feed-forward structure of a Draft layer: dense SwiGLU, Qwen3-MoE or Ling-MoE.

Restates the validation rules of the reference's
``aspec/config/draft_structure.py:21-101`` and ``aspec/config/ling_structure.py:20-87``:
Qwen3-MoE is plain softmax top-k with an auxiliary load-balancing loss; Ling-MoE
is fp32 sigmoid routing with a balancing bias, group-limited top-k, a shared
expert, optional SwiGLU clamps and a router z-loss.
"""
from __future__ import annotations

from typing import Mapping

from aspec_b200.config._check import boolean, nonneg_number, pos_int

FFN_TYPES = ("dense", "qwen3_moe", "ling_moe")
_LING_ONLY = ("router_z_loss_coef", "moe_router_bias_update_rate", "bias_zero_mean_update",
              "expert_swiglu_limit_list", "share_expert_swiglu_limit_list")
_MOE_ONLY = ("num_experts_per_tok", "moe_intermediate_size", "router_aux_loss_coef",
             "shared_expert_intermediate_size", "moe_shared_expert_intermediate_size",
             "num_shared_experts", "n_shared_experts", "moe_router_enable_expert_bias")


def _ling(raw: Mapping, common: dict) -> dict:
    what = "ling_moe"
    experts, top_k = common["num_experts"], common["num_experts_per_tok"]
    groups = pos_int(raw, "n_group", 1, what=what)
    group_topk = pos_int(raw, "topk_group", groups, what=what)
    if experts % groups or experts // groups < 2:
        raise ValueError("ling_moe group scoring requires at least two experts per equal-sized group")
    if group_topk > groups or top_k > group_topk * (experts // groups):
        raise ValueError("ling_moe Top-K exceeds the selected groups' expert capacity")
    if not common["norm_topk_prob"]:
        raise ValueError("ling_moe uses normalized routing (Top-1 retains its sigmoid score)")
    if common["router_aux_loss_coef"] != 0:
        raise ValueError("ling_moe uses bias balancing, not router_aux_loss_coef")
    for key, expected in (("topk_method", "noaux_tc"), ("score_function", "sigmoid"),
                          ("scoring_func", "sigmoid"), ("router_dtype", "fp32")):
        if raw.get(key, expected) != expected:
            raise ValueError(f"ling_moe requires {key}={expected}")
    if raw.get("mlp_only_layers") or raw.get("decoder_sparse_step", 1) != 1 or raw.get("first_k_dense_replace", 0):
        raise ValueError("ling_moe Draft uses MoE in every decoder layer")
    if raw.get("hidden_act", "silu") != "silu" or raw.get("scale_router_input", False) or raw.get("up_proj_norm", False):
        raise ValueError("ling_moe requires unscaled router input and plain SwiGLU")
    for alias in ("shared_expert_intermediate_size", "n_shared_experts"):
        if raw.get(alias):
            raise ValueError(f"ling_moe uses canonical shared expert fields, not {alias}")
    shared = raw.get("num_shared_experts", 1)
    if isinstance(shared, bool) or not isinstance(shared, int) or shared < 0:
        raise ValueError("ling_moe num_shared_experts must be a non-negative integer")
    width = pos_int(raw, "moe_shared_expert_intermediate_size", what=what) if shared else 0
    if not shared and raw.get("moe_shared_expert_intermediate_size", 0) not in (None, 0):
        raise ValueError("ling_moe shared expert width requires num_shared_experts > 0")
    enabled = boolean(raw, "moe_router_enable_expert_bias", True, what=what)
    zero_mean = boolean(raw, "bias_zero_mean_update", True, what=what)
    rate = nonneg_number(raw, "moe_router_bias_update_rate", 0.001 if enabled else 0.0, what=what)
    if not enabled and rate:
        raise ValueError("ling_moe bias update rate requires enabled expert bias")
    scale = nonneg_number(raw, "routed_scaling_factor", 2.5, what=what, positive=True)
    limits = {}
    n_layers = raw.get("num_hidden_layers")
    for key in ("expert_swiglu_limit_list", "share_expert_swiglu_limit_list"):
        values = raw.get(key)
        if values is None:
            values = [0.0] * pos_int(raw, "num_hidden_layers", what=what)
        if not isinstance(values, (list, tuple)) or len(values) != n_layers:
            raise ValueError(f"ling_moe {key} must have one limit per Draft layer")
        limits[key] = [nonneg_number({"v": v}, "v", 0.0, what=f"ling_moe {key}") for v in values]
    return {**common, "num_shared_experts": shared, "moe_shared_expert_intermediate_size": width,
            "n_group": groups, "topk_group": group_topk, "routed_scaling_factor": scale,
            "router_dtype": "fp32", "score_function": "sigmoid", "scoring_func": "sigmoid",
            "topk_method": "noaux_tc", "moe_router_enable_expert_bias": enabled,
            "moe_router_bias_update_rate": rate, "bias_zero_mean_update": zero_mean,
            "router_z_loss_coef": nonneg_number(raw, "router_z_loss_coef", 3.5e-6, what=what),
            **limits}


def resolve_ffn_policy(raw: Mapping) -> dict:
    if raw.get("architectures") == ["LlamaForCausalLMEagle4"]:
        from aspec_b200.config.eagle4 import eagle4_structure
        return eagle4_structure(raw)
    ffn = raw.get("ffn_type", "dense")
    if ffn not in FFN_TYPES:
        raise ValueError(f"Unsupported Draft ffn_type={ffn!r}")
    if ffn != "ling_moe" and any(raw.get(k) for k in _LING_ONLY):
        raise ValueError("Ling training settings require explicit ffn_type=ling_moe")
    experts = raw.get("num_experts", 0)
    if ffn == "dense":
        if experts != 0 or any(raw.get(k) not in (None, 0) for k in _MOE_ONLY):
            raise ValueError("MoE settings require explicit ffn_type=qwen3_moe or ling_moe")
        if raw.get("hidden_act", "silu") not in ("silu", "gelu", "relu", "gelu_pytorch_tanh"):
            raise ValueError(f"Unsupported Dense hidden_act={raw.get('hidden_act')!r}")
        return {"ffn_type": "dense"}
    common = {"ffn_type": ffn}
    for key in ("num_experts", "num_experts_per_tok", "moe_intermediate_size"):
        common[key] = pos_int(raw, key, what="MoE Draft")
    if common["num_experts_per_tok"] > common["num_experts"]:
        raise ValueError("MoE Draft num_experts_per_tok exceeds num_experts")
    common["norm_topk_prob"] = boolean(raw, "norm_topk_prob", True, what="MoE Draft")
    alpha = raw.get("router_aux_loss_coef")
    if alpha is None:
        alpha = 0.0 if ffn == "ling_moe" else 0.001
    common["router_aux_loss_coef"] = nonneg_number({"a": alpha}, "a", 0.0, what="MoE Draft router_aux_loss_coef")
    if ffn == "ling_moe":
        return _ling(raw, common)
    for key in ("shared_expert_intermediate_size", "moe_shared_expert_intermediate_size",
                "num_shared_experts", "n_shared_experts", "n_group", "topk_group"):
        if raw.get(key, 0):
            raise ValueError(f"qwen3_moe does not implement {key}")
    if raw.get("mlp_only_layers") or raw.get("decoder_sparse_step", 1) != 1:
        raise ValueError("qwen3_moe Draft uses MoE in every decoder layer")
    if raw.get("hidden_act", "silu") != "silu":
        raise ValueError("qwen3_moe Draft requires SwiGLU hidden_act=silu")
    if raw.get("topk_method", "greedy") != "greedy":
        raise ValueError("qwen3_moe Draft implements ungrouped greedy Top-K routing")
    for key in ("score_function", "scoring_func"):
        if raw.get(key, "softmax") != "softmax":
            raise ValueError(f"qwen3_moe requires {key}=softmax")
    if raw.get("moe_router_enable_expert_bias", False) or raw.get("routed_scaling_factor", 1.0) != 1.0:
        raise ValueError("qwen3_moe does not implement expert bias or routed scaling")
    return common


def checkpoint_ffn_policy(checkpoint_dir, topology: Mapping):
    """Routing semantics recorded with a checkpoint (falls back to its saved draft config)."""
    recorded = topology.get("draft_ffn_policy")
    if recorded is not None:
        return recorded
    if checkpoint_dir is not None:
        import json
        from pathlib import Path
        saved = Path(checkpoint_dir) / "draft_config.json"
        if saved.is_file():
            return resolve_ffn_policy(json.loads(saved.read_text()))
    return None
