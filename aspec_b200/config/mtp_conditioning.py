"""MTP-prefix conditioning of DFlash/DSpark drafts: a frozen native MTP predictor supplies the
first block token (``mode=token``) or a hidden feature fused at the anchor (``mode=hidden``).
Restates ``aspec/config/mtp_conditioning.py`` of the reference."""
from __future__ import annotations

import copy
from typing import Mapping


def resolve_mtp_conditioning(raw: Mapping):
    policy = raw.get("mtp_conditioning")
    if policy is None:
        return None
    if not isinstance(policy, Mapping) or set(policy) != {"mode", "native_config"}:
        raise ValueError("mtp_conditioning requires exactly mode and native_config")
    if policy["mode"] not in ("token", "hidden"):
        raise ValueError("MTP conditioning mode must be token or hidden")
    arch = raw.get("architectures")
    if (arch and arch[0] not in ("DFlashDraftModel", "DSparkDraftModel", "Qwen3DSparkModel")) \
            or raw.get("model_type") in ("dflash2", "k3_dspark", "qwen3_dflash2"):
        raise ValueError("MTP conditioning currently requires DFlash or DSpark full GQA")
    if not isinstance(policy["native_config"], Mapping):
        raise ValueError("MTP conditioning native_config must be a native config mapping")
    from aspec_b200.config.draft_config import NativeMTPConfig
    native = NativeMTPConfig(native_config=policy["native_config"]).native_config
    if (raw.get("ffn_type", "dense") != "dense" or raw.get("attention_mode", "gqa") != "gqa"
            or raw.get("is_causal", False)
            or any(kind != "full_attention" for kind in raw.get("layer_types", []))):
        raise ValueError("MTP conditioning currently requires Dense bidirectional full GQA Drafts")
    if native.get("attention_dropout", 0):
        raise ValueError("Frozen MTP conditioning requires zero attention dropout")
    for name, expected in (("hidden_size", raw.get("target_hidden_size")),
                           ("vocab_size", raw.get("vocab_size")),
                           ("num_hidden_layers", raw.get("target_num_hidden_layers"))):
        if native.get(name) != expected:
            raise ValueError(f"MTP native {name} disagrees with its Target/Draft binding")
    if raw.get("hidden_size") != native["hidden_size"]:
        raise ValueError("MTP conditioning requires the same frozen Target embedding width")
    if "full_attention" not in native.get("layer_types", []):
        raise ValueError("MTP native config must identify its full-attention predictor")
    return {"mode": policy["mode"], "native_config": copy.deepcopy(native)}


def mtp_conditioning_semantics(raw: Mapping):
    policy = resolve_mtp_conditioning(raw)
    if policy is None:
        return None
    return {**policy, "prefix_layout": "dual_anchor",
            "first_candidate": "teacher_forced_in_training_native_mtp_in_proposals",
            "target_context": "strictly_before_original_anchor",
            "prediction_state": "target_h[a-1]_and_token_x[a]_predict_x[a+1]",
            "feature_computation": "frozen_draft_side_native_mtp",
            "feature_stage": "native_predictor_post_norm",
            "fusion": "zero_initialized_embedding_residual" if policy["mode"] == "hidden" else None,
            "frozen": ["native_mtp", "target_embedding", "target_lm_head"]}
