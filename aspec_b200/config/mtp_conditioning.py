"""Conditioning a block Draft on a frozen native MTP predictor.

A DFlash / DSpark Draft may carry ``mtp_conditioning: {mode, native_config}``: the predictor that ships with the Target
(its native multi-token-prediction layer, frozen) supplies the first token of every block (``mode: token``) or, in
addition, its post-norm hidden state, fused into the anchor's embedding (``mode: hidden``).  This module checks that a
raw Draft configuration may use the feature and derives the description that exports record
(reference: aspec/config/mtp_conditioning.py).
"""
from __future__ import annotations

import copy
from typing import Mapping, Optional

MODES = ("token", "hidden")
_BLOCK_DRAFTS = ("DFlashDraftModel", "DSparkDraftModel", "Qwen3DSparkModel")
_OTHER_FAMILIES = ("dflash2", "qwen3_dflash2", "k3_dspark")
# native predictor field -> Draft field it must equal
_BINDINGS = {"hidden_size": "target_hidden_size", "vocab_size": "vocab_size", "num_hidden_layers": "target_num_hidden_layers"}


def _refuse(reason: str) -> None:
    raise ValueError(f"mtp_conditioning: {reason}")


def _draft_is_plain_block_model(raw: Mapping) -> bool:
    """Dense feed-forward, bidirectional full GQA attention in every layer: the only Draft shape the prefix supports."""
    architecture = (raw.get("architectures") or [None])[0]
    if architecture is not None and architecture not in _BLOCK_DRAFTS:
        return False
    if raw.get("model_type") in _OTHER_FAMILIES:
        return False
    layers_ok = all(kind == "full_attention" for kind in raw.get("layer_types", ()))
    return (layers_ok and raw.get("ffn_type", "dense") == "dense" and raw.get("attention_mode", "gqa") == "gqa"
            and not raw.get("is_causal", False))


def resolve_mtp_conditioning(raw: Mapping) -> Optional[dict]:
    """``None`` when the Draft is unconditioned, else ``{"mode", "native_config"}`` with the native config normalised."""
    spec = raw.get("mtp_conditioning")
    if spec is None:
        return None
    if not isinstance(spec, Mapping) or sorted(spec) != ["mode", "native_config"]:
        _refuse("expected exactly the keys mode and native_config")
    if spec["mode"] not in MODES:
        _refuse(f"mode must be one of {MODES}")
    if not isinstance(spec["native_config"], Mapping):
        _refuse("native_config must be the predictor's configuration mapping")
    if not _draft_is_plain_block_model(raw):
        _refuse("only dense DFlash / DSpark Drafts with bidirectional full GQA attention can be conditioned")
    from aspec_b200.config.draft_config import NativeMTPConfig
    native = NativeMTPConfig(native_config=spec["native_config"]).native_config
    if native.get("attention_dropout", 0):
        _refuse("the frozen predictor must run without attention dropout")
    if "full_attention" not in native.get("layer_types", ()):
        _refuse("the native config does not mark its full-attention predictor layer")
    for native_field, draft_field in _BINDINGS.items():
        if native.get(native_field) != raw.get(draft_field):
            _refuse(f"native {native_field}={native.get(native_field)!r} disagrees with the Draft's {draft_field}="
                    f"{raw.get(draft_field)!r}")
    if raw.get("hidden_size") != native["hidden_size"]:
        _refuse("the Draft must share the Target's embedding width (the frozen embedding is used by both)")
    return {"mode": spec["mode"], "native_config": copy.deepcopy(native)}


def mtp_conditioning_semantics(raw: Mapping) -> Optional[dict]:
    """What an export states about the conditioning, so that a consumer can check it implements the same thing."""
    resolved = resolve_mtp_conditioning(raw)
    if resolved is None:
        return None
    description = {
        "prefix_layout": "dual_anchor",
        "first_candidate": "teacher_forced_in_training_native_mtp_in_proposals",
        "target_context": "strictly_before_original_anchor",
        "prediction_state": "target_h[a-1]_and_token_x[a]_predict_x[a+1]",
        "feature_computation": "frozen_draft_side_native_mtp",
        "feature_stage": "native_predictor_post_norm",
        "fusion": "zero_initialized_embedding_residual" if resolved["mode"] == "hidden" else None,
        "frozen": ["native_mtp", "target_embedding", "target_lm_head"],
    }
    return {**resolved, **description}
