"""Attention policy of a Draft network, resolved from its JSON config.

Pure functions: JSON mapping in, normalised policy dict out, ``ValueError`` on
anything inconsistent.  The rules restate the behaviour of the reference's
``aspec/config/draft_attention.py:21-467``:

* physical head layout: MHA / MQA / GQA, or materialised MLA
  (``qk_nope + qk_rope`` query/key width, separate value width);
* per-layer schedule ``layer_types`` in {full, sliding, compressed-sparse (CSA),
  qwen-sparse (QSA), deepseek-sparse (DSA)}; the three sparse families cannot be
  mixed and each is staged ``dense -> indexer_warmup -> sparse``;
* window semantics depend on the algorithm: EAGLE = causal TTT, DFlash2 =
  query-relative, DFlash/DSpark = anchor-context (the window is measured from
  the anchor, shared by the whole block).
"""
from __future__ import annotations

import math
from typing import Mapping

from aspec_b200.config._check import nonneg_number, pos_int

LAYER_KINDS = (
    "full_attention",
    "sliding_attention",
    "compressed_sparse_attention",
    "qwen_sparse_attention",
    "deepseek_sparse_attention",
)
STAGES = ("dense", "indexer_warmup", "sparse")
_EAGLE_ARCHS = (["LlamaForCausalLMEagle3"], ["LlamaForCausalLMEagle4"], ["Eagle3DeepseekV2ForCausalLM"])
_MLA_ARCHS = (["K3DSparkModel"], ["Eagle3DeepseekV2ForCausalLM"])
DEFAULT_WORKSPACE = 2 * 1024 * 1024 * 1024      # transient budget of the sparse stages' row chunks; sized for a 180 GB GPU


def resolve_head_layout(raw: Mapping) -> dict:
    hidden = pos_int(raw, "hidden_size", 4096)
    hq = pos_int(raw, "num_attention_heads", 32)
    if raw.get("model_type") == "k3_dspark" or raw.get("architectures") in _MLA_ARCHS:
        hkv = pos_int(raw, "num_key_value_heads", hq)
        if hkv != hq:
            raise ValueError("Materialized MLA requires num_key_value_heads == num_attention_heads "
                             "after latent KV expansion")
        nope = pos_int(raw, "qk_nope_head_dim", 128)
        rope = pos_int(raw, "qk_rope_head_dim", 64)
        if rope % 2:
            raise ValueError("Draft qk_rope_head_dim must be even for rotary attention")
        q_rank = raw.get("q_lora_rank", 1536)
        if q_rank is not None:
            q_rank = pos_int({"q_lora_rank": q_rank}, "q_lora_rank")
        return {
            "type": "mla_materialized", "query_heads": hq, "key_value_heads": hkv,
            "query_heads_per_key_value_head": 1, "head_dim": nope + rope,
            "head_dim_source": "qk_nope_head_dim+qk_rope_head_dim",
            "qk_nope_head_dim": nope, "qk_rope_head_dim": rope,
            "value_head_dim": pos_int(raw, "v_head_dim", 128), "q_lora_rank": q_rank,
            "kv_lora_rank": pos_int(raw, "kv_lora_rank", 512),
            "latent_kv_materialized_before_attention": True,
        }
    hkv = pos_int(raw, "num_key_value_heads", 8)
    if hq % hkv:
        raise ValueError("Draft num_attention_heads must be divisible by num_key_value_heads; "
                         f"got {hq} and {hkv}")
    if raw.get("head_dim") is None:
        if hidden % hq:
            raise ValueError("Draft hidden_size must be divisible by num_attention_heads when "
                             f"head_dim is omitted; got {hidden} and {hq}")
        head_dim, source = hidden // hq, "hidden_size/num_attention_heads"
    else:
        head_dim, source = pos_int(raw, "head_dim"), "explicit"
    if head_dim % 2:
        raise ValueError(f"Draft head_dim must be even for rotary attention, got {head_dim}")
    kind = "mha" if hq == hkv else "mqa" if hkv == 1 else "gqa"
    return {"type": kind, "query_heads": hq, "key_value_heads": hkv,
            "query_heads_per_key_value_head": hq // hkv, "head_dim": head_dim,
            "head_dim_source": source}


def _stage(raw: Mapping, key: str) -> str:
    stage = raw.get(key, "dense")
    if stage not in STAGES:
        raise ValueError(f"Draft {key} must be dense, indexer_warmup or sparse")
    return stage


def _loss_coef(raw: Mapping, key: str, stage: str) -> float:
    coef = nonneg_number(raw, key, 1.0)
    if stage == "indexer_warmup" and coef == 0:
        raise ValueError(f"Draft {key} must be positive during indexer_warmup")
    return coef


def _csa(raw: Mapping, ratios: list) -> dict:
    stage = _stage(raw, "csa_training_stage")
    return {
        "variant": "csa", "training_stage": stage, "compress_ratios": ratios,
        "index_topk": pos_int(raw, "index_topk", 64),
        "index_n_heads": pos_int(raw, "index_n_heads", 8),
        "index_head_dim": pos_int(raw, "index_head_dim", 64),
        "indexer_loss_coef": _loss_coef(raw, "csa_indexer_loss_coef", stage),
        "workspace_bytes": pos_int(raw, "csa_workspace_bytes", DEFAULT_WORKSPACE),
        "compress_rope_theta": nonneg_number(
            {"compress_rope_theta": raw.get("compress_rope_theta", raw.get("rope_theta", 10000.0))},
            "compress_rope_theta", 10000.0, positive=True),
        "indexer_input_detached": True, "cross_layer_reuse": False,
    }


def _qsa(raw: Mapping) -> dict:
    stage = _stage(raw, "qsa_training_stage")
    ratio = pos_int(raw, "qsa_compress_ratio", 4)
    if ratio < 2:
        raise ValueError("Draft qsa_compress_ratio must be at least two")
    budget = pos_int(raw, "qsa_token_budget", 2048)
    if budget % ratio:
        raise ValueError("Draft qsa_token_budget must be divisible by qsa_compress_ratio")
    head_dim = pos_int(raw, "qsa_index_head_dim", 128)
    rope_dim = pos_int(raw, "qsa_rope_dim", 64)
    if rope_dim > head_dim or rope_dim % 2:
        raise ValueError("Draft qsa_rope_dim must be even and no larger than qsa_index_head_dim")
    return {
        "variant": "qsa", "training_stage": stage, "token_budget": budget,
        "compress_ratio": ratio, "block_topk": budget // ratio,
        "index_n_heads": pos_int(raw, "qsa_index_n_heads", 4), "index_head_dim": head_dim,
        "rope_dim": rope_dim,
        "rope_theta": nonneg_number(
            {"qsa_rope_theta": raw.get("qsa_rope_theta", raw.get("rope_theta", 10000.0))},
            "qsa_rope_theta", 10000.0, positive=True),
        "indexer_loss_coef": _loss_coef(raw, "qsa_indexer_loss_coef", stage),
        "workspace_bytes": pos_int(raw, "qsa_workspace_bytes", DEFAULT_WORKSPACE),
        "indexer_input_detached": False, "cross_layer_reuse": False,
        "draft_block_index_reuse": True, "sparse_core_backend": "selected_varlen",
    }


def _dsa(raw: Mapping) -> dict:
    stage = _stage(raw, "dsa_training_stage")
    head_dim = pos_int(raw, "dsa_index_head_dim", 128)
    rope_dim = pos_int(raw, "dsa_rope_dim", min(64, head_dim))
    if rope_dim % 2 or rope_dim > head_dim:
        raise ValueError("Draft dsa_rope_dim must be even and no larger than dsa_index_head_dim")
    return {
        "variant": "dsa", "training_stage": stage,
        "token_budget": pos_int(raw, "dsa_token_budget", 2048),
        "index_n_heads": pos_int(raw, "dsa_index_n_heads", 8), "index_head_dim": head_dim,
        "q_lora_rank": pos_int(raw, "dsa_q_lora_rank", 128), "rope_dim": rope_dim,
        "rope_theta": nonneg_number(
            {"dsa_rope_theta": raw.get("dsa_rope_theta", raw.get("rope_theta", 10000.0))},
            "dsa_rope_theta", 10000.0, positive=True),
        "indexer_loss_coef": _loss_coef(raw, "dsa_indexer_loss_coef", stage),
        "workspace_bytes": pos_int(raw, "dsa_workspace_bytes", DEFAULT_WORKSPACE),
        "indexer_input_detached": True, "cross_layer_reuse": False,
        "draft_block_index_reuse": False, "sparse_core_backend": "selected_varlen",
    }


_CSA_KEYS = ("csa_training_stage", "index_topk", "index_n_heads", "index_head_dim",
             "csa_indexer_loss_coef", "csa_workspace_bytes", "compress_rope_theta")
_QSA_KEYS = ("qsa_training_stage", "qsa_token_budget", "qsa_compress_ratio", "qsa_index_n_heads",
             "qsa_index_head_dim", "qsa_rope_dim", "qsa_rope_theta", "qsa_indexer_loss_coef",
             "qsa_workspace_bytes")
_DSA_KEYS = ("dsa_training_stage", "dsa_token_budget", "dsa_index_n_heads", "dsa_index_head_dim",
             "dsa_q_lora_rank", "dsa_rope_dim", "dsa_rope_theta", "dsa_indexer_loss_coef",
             "dsa_workspace_bytes")


def resolve_attention_policy(raw: Mapping) -> dict:
    layers = raw.get("num_hidden_layers", 1)
    if isinstance(layers, bool) or not isinstance(layers, int) or layers < 1:
        raise ValueError("Draft num_hidden_layers must be a positive integer")
    window = raw.get("sliding_window")
    if window is not None:
        try:
            window = pos_int({"w": window}, "w")
        except ValueError:
            raise ValueError("Draft sliding_window must be a positive integer or null") from None
    ratios = raw.get("compress_ratios")
    if ratios is not None:
        if not isinstance(ratios, (list, tuple)) or len(ratios) != layers:
            raise ValueError("Draft compress_ratios must contain one entry per decoder layer")
        if any(isinstance(r, bool) or not isinstance(r, int) or r < 0 for r in ratios):
            raise ValueError("Draft compress_ratios must contain non-negative integers")
        ratios = list(ratios)
    legacy = raw.get("use_sliding_window")
    if legacy is not None and not isinstance(legacy, bool):
        raise ValueError("Draft use_sliding_window must be boolean")
    if raw.get("max_window_layers") is not None:
        raise ValueError("Use explicit Draft layer_types instead of max_window_layers")
    schedule = raw.get("layer_types")
    if schedule is None:
        if ratios is not None and any(ratios):
            if window is None:
                raise ValueError("CSA Draft requires sliding_window for its local attention branch")
            schedule = ["compressed_sparse_attention" if r else "sliding_attention" for r in ratios]
        else:
            on = window is not None and legacy is not False
            schedule = ["sliding_attention" if on else "full_attention"] * layers
    if not isinstance(schedule, (list, tuple)) or len(schedule) != layers:
        raise ValueError("Draft layer_types must contain one entry per decoder layer")
    if any(kind not in LAYER_KINDS for kind in schedule):
        raise ValueError("Draft layer_types supports " + ", ".join(LAYER_KINDS) + " only")
    windowed = any(k in ("sliding_attention", "compressed_sparse_attention") for k in schedule)
    active = {name: kind in schedule for name, kind in
              (("csa", "compressed_sparse_attention"), ("qsa", "qwen_sparse_attention"),
               ("dsa", "deepseek_sparse_attention"))}
    if sum(active.values()) > 1:
        raise ValueError("Draft CSA, QSA and DSA cannot be mixed in one layer schedule")
    if windowed and window is None:
        raise ValueError("Draft sliding/CSA attention requires sliding_window")
    if legacy is not None and legacy != windowed:
        raise ValueError("Draft use_sliding_window conflicts with layer_types/sliding_window")
    if ratios is None:
        ratios = [0] * layers
    for i, (kind, ratio) in enumerate(zip(schedule, ratios)):
        if kind == "compressed_sparse_attention":
            if ratio < 2:
                raise ValueError(f"Draft CSA layer {i} requires compress_ratio >= 2")
            if ratio != 4:
                raise ValueError(f"Draft CSA layer {i} currently requires compress_ratio=4")
        elif ratio:
            raise ValueError(f"Draft compress_ratios[{i}] is only valid for compressed_sparse_attention")
    for name, keys in (("csa", _CSA_KEYS), ("qsa", _QSA_KEYS), ("dsa", _DSA_KEYS)):
        if not active[name] and any(raw.get(k) is not None for k in keys):
            raise ValueError(f"{name.upper()} settings require a matching sparse Draft layer type")
    arch = raw.get("architectures")
    if arch in _EAGLE_ARCHS:
        semantics, block = "causal_ttt", "causal_ttt_cache"
    elif arch == ["NativeMTPDraftModel"]:
        semantics, block = "anchor_context", "causal_native_mtp"
    elif arch == ["DFlash2DraftModel"]:
        causal = raw.get("is_causal")
        semantics = "query_relative"
        block = ["causal" if (causal if causal is not None else k == "sliding_attention")
                 else "bidirectional" for k in schedule]
    else:
        semantics, block = "anchor_context", "bidirectional"
    policy = {
        "sliding_window": window, "layer_types": list(schedule), "compress_ratios": ratios,
        "csa": _csa(raw, ratios) if active["csa"] else None,
        "qsa": _qsa(raw) if active["qsa"] else None,
        "context_windows": [window if k in ("sliding_attention", "compressed_sparse_attention")
                            else None for k in schedule],
        "window_semantics": semantics, "draft_block_attention": block,
    }
    if active["dsa"]:
        if raw.get("model_type") in ("k3_dspark", "qwen3_dflash2"):
            raise NotImplementedError("DSA is not integrated with materialized MLA or DFlash2")
        policy["dsa"] = _dsa(raw)
    return policy


def context_shard_alignment(policy: Mapping) -> int:
    """Minimum alignment of a context-parallel shard boundary (lcm of compression ratios)."""
    ratios = []
    if isinstance(policy.get("csa"), Mapping):
        ratios += [int(r) for r in policy["csa"]["compress_ratios"] if r]
    if isinstance(policy.get("qsa"), Mapping):
        ratios.append(int(policy["qsa"]["compress_ratio"]))
    return math.lcm(*ratios) if ratios else 1


def thd_contract(policy: Mapping, *, frozen_backbone: bool = False) -> dict:
    """Which packed-sequence kernel family each layer uses (fixed interval mask vs selected keys)."""
    frozen = frozen_backbone or any(
        (policy.get(k) or {}).get("training_stage") == "indexer_warmup" for k in ("csa", "qsa", "dsa"))
    fam = {"compressed_sparse_attention": "csa", "qwen_sparse_attention": "qsa",
           "deepseek_sparse_attention": "dsa"}
    modes = sorted({
        "varlen_selected" if (fam.get(kind) and (policy.get(fam[kind]) or {}).get("training_stage") == "sparse")
        else "interval" for kind in policy["layer_types"]})
    return {"qkv_format": "thd", "kernel_backend": "sm100_flash",
            "kernel_mode": modes[0] if len(modes) == 1 else "mixed",
            "backward_strategy": "not_required_frozen_backbone" if frozen else "sm100_flash_bwd",
            "kernel_modes": modes}
