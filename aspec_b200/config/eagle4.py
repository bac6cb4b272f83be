"""EAGLE4 policy: one recurrent decoder layer plus a low-rank candidate head.

Behavioural restatement of the reference's ``aspec/config/eagle4.py``: stages
``draft`` / ``candidate_head``; the candidate head is ``up(down(h))`` of a given
rank that retrieves ``num_candidates`` tokens and is trained with a top-K
teacher forward KL; the optional MoE uses sigmoid / auxiliary-loss-free routing.
"""
from __future__ import annotations

import math
from typing import Mapping


def _posint(name, value, limit=None):
    if type(value) is not int or value <= 0 or (limit is not None and value > limit):
        raise ValueError(f"EAGLE4 {name} must be a positive integer within its tensor extent")
    return value


def eagle4_policy(raw: Mapping) -> dict:
    if raw.get("num_hidden_layers", 1) != 1:
        raise ValueError("EAGLE4 recurrent Draft requires one decoder layer")
    stage = raw.get("eagle4_training_stage", "draft")
    if stage not in ("draft", "candidate_head"):
        raise ValueError("EAGLE4 stage must be draft or candidate_head")
    if (raw.get("draft_vocab_size") or raw["vocab_size"]) != raw["vocab_size"]:
        raise ValueError("EAGLE4 candidate retrieval requires the full target vocabulary")
    if raw.get("lm_head_rank_divisor"):
        raise ValueError("EAGLE4 needs a dense exact head, not lm_head_rank_divisor")
    head = raw.get("efficient_lm_head_config")
    if not isinstance(head, Mapping) or head.get("type") != "low_rank":
        raise ValueError("EAGLE4 requires efficient_lm_head_config.type=low_rank")
    rank = _posint("rank", head.get("rank"), min(raw["hidden_size"], raw["vocab_size"]))
    cands = _posint("num_candidates", head.get("num_candidates"), raw["vocab_size"])
    teacher_k = _posint("candidate_teacher_top_k", raw.get("candidate_teacher_top_k") or cands, raw["vocab_size"])
    chunk = _posint("candidate_loss_chunk_size", raw.get("candidate_loss_chunk_size") or 128)
    for name in ("fc_norm", "norm_output", "attn_norm", "enable_post_mlp_norm", "enable_moe", "use_rope"):
        if name in raw and not isinstance(raw[name], bool):
            raise ValueError(f"EAGLE4 {name} must be boolean")
    for name in ("enable_2hs", "enable_defa", "bias", "attention_bias", "mlp_bias"):
        if raw.get(name):
            raise ValueError(f"EAGLE4 does not implement {name}")
    if raw.get("rope_is_neox_style", True) is False and raw.get("use_rope", True):
        raise ValueError("EAGLE4 interleaved RoPE requires a matching attention implementation")
    return {"stage": stage, "rank": rank, "num_candidates": cands, "teacher_top_k": teacher_k,
            "loss_chunk_size": chunk, "candidate_objective": "frozen_draft_topk_forward_kl",
            "initialization": "randomized_truncated_svd"}


def eagle4_training_policy(raw: Mapping) -> dict:
    """Identity used for exact resume: the chunk size is a workspace bound, not semantics."""
    policy = eagle4_policy(raw)
    policy.pop("loss_chunk_size")
    return policy


def eagle4_structure(raw: Mapping) -> dict:
    if not raw.get("enable_moe", False):
        if raw.get("ffn_type", "dense") != "dense" or any(
                raw.get(k, 0) for k in ("n_routed_experts", "n_shared_experts", "num_experts_per_tok", "moe_intermediate_size")):
            raise ValueError("EAGLE4 MoE settings require enable_moe=true")
        return {"ffn_type": "dense"}
    if raw.get("ffn_type", "eagle4_moe") not in ("dense", "eagle4_moe"):
        raise ValueError("EAGLE4 uses its explicit router, not another FFN policy")
    arch = raw.get("moe_architecture", "sparse_swiglu")
    if arch not in ("sparse_swiglu", "nemotron_latent_relu2"):
        raise ValueError(f"Unsupported EAGLE4 MoE architecture: {arch!r}")
    n, k = raw.get("n_routed_experts"), raw.get("num_experts_per_tok")
    group = raw.get("n_group", 1) or 1
    selected = raw.get("topk_group", raw.get("n_group", 1)) or 1
    for name, value in (("n_routed_experts", n), ("num_experts_per_tok", k),
                        ("moe_intermediate_size", raw.get("moe_intermediate_size")),
                        ("n_group", group), ("topk_group", selected)):
        if type(value) is not int or value <= 0:
            raise ValueError(f"EAGLE4 {name} must be positive")
    if k > n or n % group or selected > group or k > n // group * selected or (group > 1 and n // group < 2):
        raise ValueError("EAGLE4 MoE group/top-k geometry is invalid")
    shared = raw.get("n_shared_experts", 0) or 0
    if type(shared) is not int or shared < 0:
        raise ValueError("EAGLE4 n_shared_experts must be non-negative")
    if raw.get("scoring_func", "sigmoid") != "sigmoid" or raw.get("topk_method", "noaux_tc") != "noaux_tc":
        raise ValueError("EAGLE4 MoE requires sigmoid/noaux_tc routing")
    if type(raw.get("norm_topk_prob", True)) is not bool:
        raise ValueError("EAGLE4 norm_topk_prob must be boolean")
    if raw.get("hidden_act", "silu") != ("relu2" if arch == "nemotron_latent_relu2" else "silu"):
        raise ValueError("EAGLE4 MoE activation disagrees with architecture")
    rate = raw.get("expert_bias_update_rate", raw.get("moe_router_bias_update_rate", 0.001))
    scale = raw.get("routed_scaling_factor", 1.0)
    for name, value in (("expert_bias_update_rate", rate), ("routed_scaling_factor", scale)):
        if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or value < 0:
            raise ValueError(f"EAGLE4 {name} must be finite and non-negative")
    out = {"ffn_type": "eagle4_moe", "moe_architecture": arch, "n_routed_experts": n,
           "num_experts_per_tok": k, "moe_intermediate_size": raw["moe_intermediate_size"],
           "n_shared_experts": shared, "n_group": group, "topk_group": selected,
           "norm_topk_prob": raw.get("norm_topk_prob", True), "routed_scaling_factor": float(scale),
           "expert_bias_update_rate": float(rate)}
    if arch == "nemotron_latent_relu2":
        for name in ("moe_latent_size", "moe_shared_expert_intermediate_size"):
            out[name] = _posint(name, raw.get(name))
    for key in ("aux_loss_alpha", "seq_aux_loss_alpha", "load_balance_loss_alpha", "moe_seq_aux_loss_coeff"):
        if raw.get(key, 0):
            raise ValueError("EAGLE4 implements auxiliary-loss-free routing, not nonzero " + key)
    return out


def eagle4_asset_metadata(raw: Mapping, steps: int) -> dict:
    policy = eagle4_policy(raw)
    candidate = policy["stage"] == "candidate_head"
    if type(steps) is not int or steps < 0 or candidate != (steps > 0):
        raise ValueError("EAGLE4 candidate asset requires completed training; draft assets require zero candidate steps")
    return {**policy, "candidate_optimizer_steps": steps, "candidate_head_trained": candidate,
            "scope": "trained_candidate" if candidate else "draft_initialization"}
