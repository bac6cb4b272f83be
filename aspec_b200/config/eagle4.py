"""Validation and derived settings of an EAGLE4 Draft configuration.

An EAGLE4 Draft is one recurrent decoder layer (dense or mixture-of-experts feed-forward) with an exact output head
over the full Target vocabulary plus a low-rank *candidate head* ``up(down(h))`` that retrieves a short list of
tokens.  Training has two stages - ``draft`` (everything but the candidate head) and ``candidate_head`` (only the
candidate head, distilled from the frozen Draft's own top-K distribution).  The rules enforced here are those of the
reference (aspec/config/eagle4.py:28-174); they are written as small checks over the raw dictionary.
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional

STAGES = ("draft", "candidate_head")
MOE_LAYOUTS = {"sparse_swiglu": "silu", "nemotron_latent_relu2": "relu2"}      # layout -> required activation
_UNSUPPORTED_SWITCHES = ("enable_2hs", "enable_defa", "bias", "attention_bias", "mlp_bias")
_BOOLEAN_SWITCHES = ("fc_norm", "norm_output", "attn_norm", "enable_post_mlp_norm", "enable_moe", "use_rope")
_AUXILIARY_LOSSES = ("aux_loss_alpha", "seq_aux_loss_alpha", "load_balance_loss_alpha", "moe_seq_aux_loss_coeff")
_MOE_ONLY_KEYS = ("n_routed_experts", "n_shared_experts", "num_experts_per_tok", "moe_intermediate_size")


def _fail(message: str) -> None:
    raise ValueError(f"EAGLE4 configuration: {message}")


def _count(raw: Mapping, key: str, *, default: Optional[int] = None, at_most: Optional[int] = None) -> int:
    """A strictly positive ``int`` (booleans and floats are refused), optionally bounded above."""
    value: Any = raw.get(key)
    if value is None:
        value = default
    if type(value) is not int or value < 1:
        _fail(f"{key} must be a positive integer, got {value!r}")
    if at_most is not None and value > at_most:
        _fail(f"{key}={value} exceeds the tensor extent {at_most}")
    return value


def _nonnegative_number(raw: Mapping, keys, default: float) -> float:
    value = next((raw[k] for k in keys if raw.get(k) is not None), default)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or value < 0:
        _fail(f"{keys[0]} must be a finite number >= 0, got {value!r}")
    return float(value)


def eagle4_policy(raw: Mapping) -> dict:
    """Stage, candidate-head geometry and objective of the configuration (raises ``ValueError`` on a bad one)."""
    vocab, hidden = raw["vocab_size"], raw["hidden_size"]
    if raw.get("num_hidden_layers", 1) != 1:
        _fail("the recurrent Draft has exactly one decoder layer")
    stage = raw.get("eagle4_training_stage", STAGES[0])
    if stage not in STAGES:
        _fail(f"eagle4_training_stage must be one of {STAGES}")
    if raw.get("draft_vocab_size") not in (None, 0, vocab):
        _fail("candidate retrieval works on the full Target vocabulary (no pruned draft_vocab_size)")
    if raw.get("lm_head_rank_divisor"):
        _fail("the exact head is dense; lm_head_rank_divisor is not supported")
    head = raw.get("efficient_lm_head_config")
    if not isinstance(head, Mapping) or head.get("type") != "low_rank":
        _fail("efficient_lm_head_config must be {type: low_rank, rank, num_candidates}")
    for key in _BOOLEAN_SWITCHES:
        if key in raw and not isinstance(raw[key], bool):
            _fail(f"{key} must be true or false")
    enabled = [key for key in _UNSUPPORTED_SWITCHES if raw.get(key)]
    if enabled:
        _fail(f"not implemented: {', '.join(enabled)}")
    if raw.get("use_rope", True) and raw.get("rope_is_neox_style", True) is False:
        _fail("interleaved (non-NeoX) RoPE has no matching attention path")
    candidates = _count(head, "num_candidates", at_most=vocab)
    return {
        "stage": stage,
        "rank": _count(head, "rank", at_most=min(hidden, vocab)),
        "num_candidates": candidates,
        "teacher_top_k": _count(raw, "candidate_teacher_top_k", default=candidates, at_most=vocab),
        "loss_chunk_size": _count(raw, "candidate_loss_chunk_size", default=128),
        "candidate_objective": "frozen_draft_topk_forward_kl",
        "initialization": "randomized_truncated_svd",
    }


def eagle4_training_policy(raw: Mapping) -> dict:
    """What must agree for an exact resume: everything in the policy except the loss chunk (a workspace bound)."""
    return {k: v for k, v in eagle4_policy(raw).items() if k != "loss_chunk_size"}


def eagle4_structure(raw: Mapping) -> dict:
    """Feed-forward structure: ``{"ffn_type": "dense"}`` or the validated mixture-of-experts geometry."""
    if not raw.get("enable_moe", False):
        leftovers = [k for k in _MOE_ONLY_KEYS if raw.get(k, 0)]
        if leftovers or raw.get("ffn_type", "dense") != "dense":
            _fail("mixture-of-experts fields are set but enable_moe is false")
        return {"ffn_type": "dense"}
    if raw.get("ffn_type", "eagle4_moe") not in ("dense", "eagle4_moe"):
        _fail("EAGLE4 brings its own router; other ffn_type policies do not apply")
    layout = raw.get("moe_architecture", "sparse_swiglu")
    if layout not in MOE_LAYOUTS:
        _fail(f"unknown moe_architecture {layout!r}")
    if raw.get("hidden_act", "silu") != MOE_LAYOUTS[layout]:
        _fail(f"moe_architecture {layout} runs with hidden_act={MOE_LAYOUTS[layout]}")
    experts = _count(raw, "n_routed_experts")
    per_token = _count(raw, "num_experts_per_tok")
    inner = _count(raw, "moe_intermediate_size")
    groups = _count(raw, "n_group", default=1) if raw.get("n_group") else 1
    kept = _count(raw, "topk_group", default=groups) if raw.get("topk_group") else groups
    per_group, remainder = divmod(experts, groups)
    geometry_ok = (per_token <= experts and remainder == 0 and kept <= groups and per_token <= per_group * kept
                   and (groups == 1 or per_group >= 2))
    if not geometry_ok:
        _fail(f"impossible routing geometry: {experts} experts in {groups} groups, {kept} groups kept, top-{per_token}")
    shared = raw.get("n_shared_experts") or 0
    if type(shared) is not int or shared < 0:
        _fail("n_shared_experts must be an integer >= 0")
    if raw.get("scoring_func", "sigmoid") != "sigmoid" or raw.get("topk_method", "noaux_tc") != "noaux_tc":
        _fail("routing is sigmoid scoring with the bias-based (noaux_tc) selection")
    if not isinstance(raw.get("norm_topk_prob", True), bool):
        _fail("norm_topk_prob must be true or false")
    nonzero = [k for k in _AUXILIARY_LOSSES if raw.get(k, 0)]
    if nonzero:
        _fail(f"load balancing is auxiliary-loss-free; {', '.join(nonzero)} must stay 0")
    structure = {
        "ffn_type": "eagle4_moe", "moe_architecture": layout, "n_routed_experts": experts, "num_experts_per_tok": per_token,
        "moe_intermediate_size": inner, "n_shared_experts": shared, "n_group": groups, "topk_group": kept,
        "norm_topk_prob": raw.get("norm_topk_prob", True),
        "routed_scaling_factor": _nonnegative_number(raw, ("routed_scaling_factor",), 1.0),
        "expert_bias_update_rate": _nonnegative_number(raw, ("expert_bias_update_rate", "moe_router_bias_update_rate"), 1e-3),
    }
    if layout == "nemotron_latent_relu2":
        structure["moe_latent_size"] = _count(raw, "moe_latent_size")
        structure["moe_shared_expert_intermediate_size"] = _count(raw, "moe_shared_expert_intermediate_size")
    return structure


def eagle4_asset_metadata(raw: Mapping, steps: int) -> dict:
    """Export metadata: a ``candidate_head`` asset must have trained (``steps > 0``), a ``draft`` asset must not."""
    policy = eagle4_policy(raw)
    trained = policy["stage"] == "candidate_head"
    if type(steps) is not int or steps < 0 or trained != (steps > 0):
        _fail("a candidate_head asset needs completed candidate steps; a draft asset has none")
    return {**policy, "candidate_optimizer_steps": steps, "candidate_head_trained": trained,
            "scope": "trained_candidate" if trained else "draft_initialization"}
