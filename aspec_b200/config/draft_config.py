"""Draft model configuration objects (JSON <-> attribute bags with validation).

The JSON schema is the one the reference ships under ``aspec/config/*.json`` and
reads through ``AutoDraftModelConfig.from_file`` (aspec/models/draft/auto.py:66-121):
an ``architectures`` list with one registered name selects the algorithm
(aspec/config/draft_algorithm.py:19-29).  Here a config is a light attribute bag
(no ``transformers.PretrainedConfig`` machinery): ``to_dict`` returns exactly what
``save_pretrained`` writes and ``from_dict`` accepts it back.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict, Mapping

from aspec_b200.config.draft_attention import resolve_attention_policy, resolve_head_layout
from aspec_b200.config.draft_structure import resolve_ffn_policy
from aspec_b200.config.rope import resolve_rope_parameters

DRAFT_ALGORITHMS = {
    "NativeMTPDraftModel": "mtp",
    "DFlashDraftModel": "dflash",
    "DFlash2DraftModel": "dflash2",
    "DSparkDraftModel": "dspark",
    "Qwen3DSparkModel": "dspark",
    "K3DSparkModel": "dspark",
    "LlamaForCausalLMEagle3": "eagle3",
    "LlamaForCausalLMEagle4": "eagle4",
    "Eagle3DeepseekV2ForCausalLM": "eagle3",
}


def resolve_draft_algorithm(raw: Mapping) -> str:
    arch = raw.get("architectures")
    if not isinstance(arch, list) or len(arch) != 1:
        raise ValueError("Draft algorithm requires exactly one registered architecture")
    try:
        return DRAFT_ALGORITHMS[arch[0]]
    except (KeyError, TypeError):
        raise ValueError(f"Unsupported Draft algorithm architecture: {arch!r}") from None


class DraftConfig:
    """Base attribute bag.  Subclasses set ``model_type``, ``defaults`` and ``_post_init``."""

    model_type = "draft"
    defaults: Dict[str, Any] = {}

    def __init__(self, **kwargs):
        merged: Dict[str, Any] = {}
        for klass in reversed(type(self).__mro__):
            merged.update(copy.deepcopy(getattr(klass, "defaults", {})))
        merged.update(kwargs)
        merged.setdefault("model_type", self.model_type)
        merged["tie_word_embeddings"] = False
        for key, value in merged.items():
            setattr(self, key, value)
        self._post_init()

    def _post_init(self) -> None:
        pass

    # -- dict / file round trip -------------------------------------------------
    def to_dict(self) -> dict:
        return {k: copy.deepcopy(v) for k, v in vars(self).items() if not k.startswith("_")}

    @classmethod
    def from_dict(cls, raw: Mapping):
        return cls(**dict(raw))

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def save_pretrained(self, directory: str) -> None:
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, "config.json"), "w") as f:
            f.write(self.to_json_string())

    def get(self, key: str, default=None):
        return getattr(self, key, default)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.to_dict()})"

    @property
    def head_dim_resolved(self) -> int:
        return resolve_head_layout(self.to_dict())["head_dim"]


class DFlashConfig(DraftConfig):
    model_type = "dflash"
    defaults = dict(
        architectures=["DFlashDraftModel"], hidden_size=4096, intermediate_size=14336,
        num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, vocab_size=152064,
        rms_norm_eps=1e-6, max_position_embeddings=32768, rope_theta=10000.0,
        num_target_layers=5, target_hidden_size=4096, target_num_hidden_layers=36,
        target_layer_ids=None, fc_norm=False, mask_token_id=151669, ffn_type="dense",
        num_experts=0, num_experts_per_tok=None, moe_intermediate_size=None, norm_topk_prob=True,
        router_aux_loss_coef=None, hidden_act="silu", mtp_conditioning=None, attention_mode="gqa",
    )
    _mla = False

    def _post_init(self) -> None:
        raw = self.to_dict()
        self.fc_norm = bool(self.fc_norm)
        if not self._mla:
            layout = resolve_head_layout(raw)
            self.head_dim = layout["head_dim"]
        policy = resolve_attention_policy(raw)
        self.sliding_window = policy["sliding_window"]
        self.layer_types = policy["layer_types"]
        self.compress_ratios = policy["compress_ratios"]
        if policy["csa"] is not None:
            csa = policy["csa"]
            self.csa_training_stage = csa["training_stage"]
            for k in ("index_topk", "index_n_heads", "index_head_dim", "compress_rope_theta"):
                setattr(self, k, csa[k])
            self.csa_indexer_loss_coef = csa["indexer_loss_coef"]
            self.csa_workspace_bytes = csa["workspace_bytes"]
        if policy["qsa"] is not None:
            qsa = policy["qsa"]
            self.qsa_training_stage = qsa["training_stage"]
            for k in ("token_budget", "compress_ratio", "index_n_heads", "index_head_dim",
                      "rope_dim", "rope_theta", "indexer_loss_coef", "workspace_bytes"):
                setattr(self, f"qsa_{k}", qsa[k])
        if policy.get("dsa") is not None:
            dsa = policy["dsa"]
            for k in ("training_stage", "token_budget", "index_n_heads", "index_head_dim",
                      "q_lora_rank", "rope_dim", "rope_theta", "indexer_loss_coef", "workspace_bytes"):
                setattr(self, f"dsa_{k}", dsa[k])
        for key, value in resolve_ffn_policy({**raw, "num_hidden_layers": self.num_hidden_layers}).items():
            setattr(self, key, value)
        if not self._mla:
            self._rope_parameters = resolve_rope_parameters(self)
        if self.target_layer_ids is not None:
            ids = list(self.target_layer_ids)
            if len(ids) != self.num_target_layers:
                raise ValueError("target_layer_ids must list num_target_layers entries")
            self.target_layer_ids = ids
        if self.mtp_conditioning is not None:
            from aspec_b200.config.mtp_conditioning import resolve_mtp_conditioning
            self.mtp_conditioning = resolve_mtp_conditioning(self.to_dict())

    @property
    def rope_parameters_resolved(self) -> dict:
        return self._rope_parameters


class DSparkConfig(DFlashConfig):
    model_type = "qwen3_dspark"
    defaults = dict(architectures=["Qwen3DSparkModel"], markov_rank=256, markov_head_type="vanilla",
                    enable_confidence_head=True, confidence_head_with_markov=True)

    def _post_init(self) -> None:
        super()._post_init()
        if int(self.markov_rank) < 0:
            raise ValueError(f"markov_rank must be >= 0, got {self.markov_rank}")
        if self.markov_rank and str(self.markov_head_type).lower() != "vanilla":
            raise NotImplementedError(f"markov_head_type={self.markov_head_type!r} is not supported; only 'vanilla'")
        if self.enable_confidence_head and self.confidence_head_with_markov and not self.markov_rank:
            raise ValueError("confidence_head_with_markov=True requires a Markov head (markov_rank > 0).")


class K3DSparkConfig(DSparkConfig):
    """DSpark with materialised multi-head latent attention (MLA)."""
    model_type = "k3_dspark"
    defaults = dict(architectures=["K3DSparkModel"], attention_mode="mla", q_lora_rank=1536,
                    kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                    num_key_value_heads=None)
    _mla = True

    def _post_init(self) -> None:
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        layout = resolve_head_layout(self.to_dict())
        self.head_dim = layout["head_dim"]
        super()._post_init()
        self._rope_parameters = {"rope_type": "default", "rope_theta": float(self.rope_theta)}


class DFlash2Config(DFlashConfig):
    model_type = "qwen3_dflash2"
    defaults = dict(architectures=["DFlash2DraftModel"], block_size=8, conv_kernel_size=4,
                    conv_group_size=8, selector_rank=256, selector_top_k=8,
                    input_embedding_scale=1.0, output_multiplier=1.0,
                    final_logit_softcapping=None, is_causal=None)


class Eagle3Config(DraftConfig):
    """Llama-shaped EAGLE3 draft (one ``midlayer``)."""
    model_type = "llama"
    defaults = dict(
        architectures=["LlamaForCausalLMEagle3"], hidden_size=4096, intermediate_size=12288,
        num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, vocab_size=151936,
        draft_vocab_size=None, rms_norm_eps=1e-6, max_position_embeddings=40960, rope_theta=1000000.0,
        rope_scaling=None, hidden_act="silu", target_hidden_size=None, num_aux_hidden_states=3,
        target_layer_ids=None, fc_norm=False, norm_output=False, lm_head_rank_divisor=None,
        sliding_window=None, pad_token_id=0,
    )

    def _post_init(self) -> None:
        if self.draft_vocab_size is None:
            self.draft_vocab_size = self.vocab_size
        if self.target_hidden_size is None:
            self.target_hidden_size = self.hidden_size
        if self.target_layer_ids:
            self.num_aux_hidden_states = len(self.target_layer_ids)
        self.head_dim = resolve_head_layout(self.to_dict())["head_dim"]
        resolve_attention_policy(self.to_dict())


class Eagle4Config(Eagle3Config):
    model_type = "llama_eagle4"
    defaults = dict(architectures=["LlamaForCausalLMEagle4"], attn_norm=True, enable_post_mlp_norm=True,
                    use_rope=True, enable_moe=False, eagle4_training_stage="draft",
                    efficient_lm_head_config=None, candidate_teacher_top_k=None,
                    candidate_loss_chunk_size=128)

    def _post_init(self) -> None:
        super()._post_init()
        from aspec_b200.config.eagle4 import eagle4_policy, eagle4_structure
        raw = self.to_dict()
        if raw.get("candidate_teacher_top_k") is None:
            raw.pop("candidate_teacher_top_k")
        self._eagle4 = eagle4_policy(raw)
        for key, value in eagle4_structure(raw).items():
            setattr(self, key, value)

    @property
    def eagle4_policy(self) -> dict:
        return dict(self._eagle4)


class DeepseekEagleConfig(Eagle3Config):
    """EAGLE3 draft whose attention is (materialised) DeepSeek MLA."""
    model_type = "deepseek_v3"
    defaults = dict(architectures=["Eagle3DeepseekV2ForCausalLM"], q_lora_rank=1536, kv_lora_rank=512,
                    qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_key_value_heads=None,
                    n_routed_experts=0, n_shared_experts=0, num_experts_per_tok=0,
                    moe_intermediate_size=0, pretraining_tp=1)

    def _post_init(self) -> None:
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        super()._post_init()


class NativeMTPConfig(DraftConfig):
    """Native multi-token-prediction head of a Qwen3.5-style Target (one full-attention layer)."""
    model_type = "native_mtp"
    defaults = dict(architectures=["NativeMTPDraftModel"], native_config=None, mtp_steps=3)

    def _post_init(self) -> None:
        native = dict(self.native_config or {})
        native = dict(native.get("text_config", native))
        for key, default in (("hidden_size", 4096), ("intermediate_size", 12288),
                             ("num_attention_heads", 32), ("num_key_value_heads", 8),
                             ("vocab_size", 151936), ("rms_norm_eps", 1e-6),
                             ("num_hidden_layers", 36), ("rope_theta", 1000000.0),
                             ("max_position_embeddings", 40960), ("attention_dropout", 0.0)):
            native.setdefault(key, default)
        native.setdefault("head_dim", native["hidden_size"] // native["num_attention_heads"])
        native.setdefault("layer_types", ["full_attention"])
        self.native_config = native
        for key in ("hidden_size", "vocab_size", "num_attention_heads", "num_key_value_heads",
                    "intermediate_size", "rms_norm_eps", "head_dim", "rope_theta"):
            setattr(self, key, native[key])
        self.num_hidden_layers = 1
        self.target_hidden_size = native["hidden_size"]
        self.target_num_hidden_layers = native["num_hidden_layers"]


class AutoDraftModelConfig:
    """``from_file`` / ``from_dict`` registry keyed by the single ``architectures`` entry."""

    _config_mapping = {
        "LlamaForCausalLMEagle3": Eagle3Config,
        "LlamaForCausalLMEagle4": Eagle4Config,
        "Eagle3DeepseekV2ForCausalLM": DeepseekEagleConfig,
        "NativeMTPDraftModel": NativeMTPConfig,
        "DFlashDraftModel": DFlashConfig,
        "DFlash2DraftModel": DFlash2Config,
        "Qwen3DSparkModel": DSparkConfig,
        "DSparkDraftModel": DSparkConfig,
        "K3DSparkModel": K3DSparkConfig,
    }

    @classmethod
    def from_dict(cls, config: Mapping) -> DraftConfig:
        config = dict(config)
        arch = config.get("architectures")
        if arch is None:
            raise ValueError("No architectures found in the config file")
        if len(arch) != 1:
            raise ValueError("Only one architecture is supported")
        if arch[0] not in cls._config_mapping:
            raise ValueError(f"Architecture {arch[0]} not supported")
        return cls._config_mapping[arch[0]].from_dict(config)

    @classmethod
    def from_file(cls, path: str) -> DraftConfig:
        with open(path) as f:
            return cls.from_dict(json.load(f))


_SEMANTIC_FIELDS = (
    "native_config", "architectures", "hidden_size", "target_hidden_size", "intermediate_size",
    "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
    "draft_vocab_size", "hidden_act", "rms_norm_eps", "max_position_embeddings", "rope_theta",
    "rope_scaling", "rope_parameters", "target_layer_ids", "num_target_layers",
    "target_num_hidden_layers", "num_aux_hidden_states", "fc_norm", "norm_output", "mask_token_id",
    "lm_head_rank_divisor", "attention_mode", "q_lora_rank", "kv_lora_rank", "qk_nope_head_dim",
    "qk_rope_head_dim", "v_head_dim", "block_size", "conv_kernel_size", "conv_group_size",
    "selector_rank", "selector_top_k", "efficient_lm_head_config", "candidate_teacher_top_k",
    "use_rope", "attn_norm", "enable_post_mlp_norm", "input_embedding_scale", "output_multiplier",
    "final_logit_softcapping", "is_causal", "markov_rank", "enable_confidence_head",
    "confidence_head_with_markov", "mtp_conditioning",
)


def draft_model_semantics(config) -> dict:
    """The fields that define *which model* a checkpoint holds (used for exact-resume identity)."""
    raw = config if isinstance(config, Mapping) else config.to_dict()
    if raw.get("architectures") and raw["architectures"][0] in DRAFT_ALGORITHMS:
        raw = AutoDraftModelConfig.from_dict(raw).to_dict()
    raw = dict(raw)
    raw["fc_norm"] = bool(raw.get("fc_norm"))
    raw["norm_output"] = bool(raw.get("norm_output"))
    raw["lm_head_rank_divisor"] = raw.get("lm_head_rank_divisor") or None
    return {k: raw[k] for k in _SEMANTIC_FIELDS if k in raw and raw[k] is not None or k in ("fc_norm", "norm_output")}
