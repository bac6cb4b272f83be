"""DFlash-family Draft network: dual-source key/value attention over packed tokens.

Architecture (reference: aspec/models/draft/dflash.py:330-1518):

* ``context_proj: Linear(K*Dt -> D)`` + ``context_norm`` turn the ``K`` captured Target layers into
  one context feature per token, computed once and fed unchanged to every layer;
* each decoder layer attends from the draft tokens to ``cat(context, draft)`` keys/values produced
  by the *same* ``k_proj`` / ``v_proj`` for both sources, with per-head RMSNorm on q and k and
  rotate-half RoPE;
* the FFN is SwiGLU, Qwen3-MoE or Ling-MoE; ``embed_tokens`` is the Target's embedding (frozen)
  and the LM head is external.

This implementation is token-major ("THD") throughout: context ``[T, D]``, draft tokens ``[Q, D]``
and an interval table ``[Q, 4]`` describing which keys each draft row sees.  A padded batch is just
several rows concatenated with disjoint intervals.  On CUDA the layer runs on the framework's
tcgen05 GEMM (k/v and gate/up fused into one GEMM each), fused QK-norm+RoPE, interval flash
attention and SwiGLU kernels; on CPU the same code runs the fp32 reference ops.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from aspec_b200.config.draft_config import DFlashConfig
from aspec_b200.config.rope import rope_inverse_frequencies
from aspec_b200.ops.activation import swiglu
from aspec_b200.ops.attention import interval_attention
from aspec_b200.ops.fused_params import allocate_adjacent, fused_linear
from aspec_b200.ops.linear import Linear, linear
from aspec_b200.ops.norm import RMSNorm
from aspec_b200.ops.rope import RopeFrequencies, qk_norm_rope


def build_target_layer_ids(num_target_layers: int, num_hidden_layers: int) -> List[int]:
    """Evenly spaced captured layers: one -> middle; else ``round(1 + i*(L-4)/(n-1))``."""
    if num_target_layers == 1:
        return [num_hidden_layers // 2]
    span = num_hidden_layers - 4
    return [int(round(1 + i * span / (num_target_layers - 1))) for i in range(num_target_layers)]


class _Weight(nn.Module):
    """A bare ``weight`` holder so fused storage keeps reference-compatible parameter names."""

    def __init__(self, weight: nn.Parameter):
        super().__init__()
        self.weight = weight

    def forward(self, x):
        return linear(x, self.weight)


class DFlashAttention(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        d, D = self.head_dim, self.hidden_size
        self.q_proj = Linear(D, self.num_heads * d)
        kw, vw = allocate_adjacent([(self.num_kv_heads * d, D)] * 2)
        nn.init.normal_(kw, std=0.02)
        nn.init.normal_(vw, std=0.02)
        self.k_proj, self.v_proj = _Weight(kw), _Weight(vw)
        self.o_proj = Linear(self.num_heads * d, D)
        self.q_norm = RMSNorm(d, eps=config.rms_norm_eps)
        self.k_norm = RMSNorm(d, eps=config.rms_norm_eps)
        inv, self.rope_scaling = rope_inverse_frequencies(d, config.rope_parameters_resolved)
        self.rope_freqs = RopeFrequencies(inv)
        self.eps = config.rms_norm_eps
        self.scale = d ** -0.5

    def forward(self, x, ctx, q_pos, kv_pos, intervals, aux=None, attn_override=None):
        attn_override = attn_override or (aux or {}).get("attention_override")
        Q, T = x.shape[0], ctx.shape[0]
        d, hk = self.head_dim, self.num_kv_heads
        q = self.q_proj(x).view(Q, self.num_heads, d)
        kv = fused_linear(torch.cat([ctx, x], 0), [self.k_proj.weight, self.v_proj.weight])
        k = kv[:, : hk * d].reshape(T + Q, hk, d)
        v = kv[:, hk * d:].view(T + Q, hk, d)
        inv_freq = self.rope_freqs.get(x.device)
        q = qk_norm_rope(q, self.q_norm.weight, q_pos, inv_freq, self.eps, self.rope_scaling)
        k = qk_norm_rope(k, self.k_norm.weight, kv_pos, inv_freq, self.eps, self.rope_scaling)
        if isinstance(intervals, dict):
            # context parallel: k / v are this rank's context shard + own draft rows; the runtime exchanges queries and
            # partial results with the other owners
            o = intervals["cp"].attention(self.layer_idx, q, k, v, intervals["tables"], intervals["counts"], self.scale)
        elif attn_override is not None:
            o = attn_override(self, q, k, v, intervals)
        else:
            o, _ = interval_attention(q, k, v, intervals, self.scale)
        return self.o_proj(o.reshape(Q, self.num_heads * d))


class DFlashMLP(nn.Module):
    """SwiGLU ``down(silu(gate(x)) * up(x))`` with gate/up stored adjacently (one GEMM)."""

    def __init__(self, hidden_size: int, intermediate_size: int, clamp: float = 0.0):
        super().__init__()
        gw, uw = allocate_adjacent([(intermediate_size, hidden_size)] * 2)
        nn.init.normal_(gw, std=0.02)
        nn.init.normal_(uw, std=0.02)
        self.gate_proj, self.up_proj = _Weight(gw), _Weight(uw)
        self.down_proj = Linear(intermediate_size, hidden_size)
        self.clamp = clamp

    def forward(self, x):
        gu = fused_linear(x, [self.gate_proj.weight, self.up_proj.weight])
        return self.down_proj(swiglu(gu, self.clamp))


def build_ffn(config, layer_idx: int) -> nn.Module:
    kind = getattr(config, "ffn_type", "dense")
    if kind == "dense":
        return DFlashMLP(config.hidden_size, config.intermediate_size)
    if kind == "qwen3_moe":
        from aspec_b200.models.draft.moe import QwenMoE
        return QwenMoE(config)
    if kind == "ling_moe":
        from aspec_b200.models.draft.ling_moe import LingMoE
        return LingMoE(config, layer_idx)
    raise ValueError(f"unknown ffn_type {kind!r}")


class DFlashDecoderLayer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        kind = config.layer_types[layer_idx]
        if kind == "compressed_sparse_attention":
            from aspec_b200.models.draft.csa import CSAAttention
            self.self_attn = CSAAttention(config, layer_idx)
        elif kind == "qwen_sparse_attention":
            from aspec_b200.models.draft.qsa import QSAAttention
            self.self_attn = QSAAttention(config, layer_idx)
        elif kind == "deepseek_sparse_attention":
            from aspec_b200.models.draft.dsa import DSAAttention
            self.self_attn = DSAAttention(config, layer_idx)
        elif getattr(config, "attention_mode", "gqa") == "mla":
            from aspec_b200.models.draft.mla import MLAAttention
            self.self_attn = MLAAttention(config, layer_idx)
        else:
            self.self_attn = DFlashAttention(config, layer_idx)
        self.mlp = build_ffn(config, layer_idx)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, x, ctx, q_pos, kv_pos, intervals, aux=None):
        x = x + self.self_attn(self.input_layernorm(x), ctx, q_pos, kv_pos, intervals, aux=aux)
        y = self.post_attention_layernorm(x)
        y = self.mlp(y, aux=aux) if getattr(self.mlp, "wants_aux", False) else self.mlp(y)
        return x + y


class DFlashDraftModel(nn.Module):
    """``context_proj`` + ``context_norm`` + frozen ``embed_tokens`` + ``layers`` + ``final_norm``."""

    config_class = DFlashConfig
    decoder_layer_class = DFlashDecoderLayer

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.num_layers = config.num_hidden_layers
        self.num_target_layers = config.num_target_layers
        self.mask_token_id = config.mask_token_id
        self.target_layer_ids = (list(config.target_layer_ids) if config.target_layer_ids is not None
                                 else build_target_layer_ids(config.num_target_layers,
                                                             config.target_num_hidden_layers))
        dt = config.target_hidden_size
        self.fc_norm = (nn.ModuleList([RMSNorm(dt, eps=config.rms_norm_eps)
                                       for _ in range(config.num_target_layers)])
                        if config.fc_norm else None)
        self.context_proj = Linear(config.num_target_layers * dt, config.hidden_size)
        self.context_norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([self.decoder_layer_class(config, i) for i in range(self.num_layers)])
        self.final_norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.gradient_checkpointing = False
        self.freeze_embedding()
        self.mtp_fusion = self.mtp_source = None
        conditioning = getattr(config, "mtp_conditioning", None)
        if conditioning:
            from aspec_b200.models.dmtp import FrozenMTPFeatures, MTPAnchorFusion
            self.mtp_source = FrozenMTPFeatures(conditioning["native_config"])
            if conditioning["mode"] == "hidden":
                self.mtp_fusion = MTPAnchorFusion(config.hidden_size, dt, eps=config.rms_norm_eps)

    def initialize_mtp_conditioning(self, tensors) -> None:
        """Load the frozen MTP predictor from the Target checkpoint tensors (``mtp.*`` keys)."""
        if self.mtp_source is not None:
            self.mtp_source.initialize_native_weights(tensors)

    def validate_mtp_binding(self, tensors, embedding=None) -> None:
        if self.mtp_source is None:
            return
        if embedding is not None and not torch.equal(self.embed_tokens.weight.detach().cpu(),
                                                     embedding.to(self.embed_tokens.weight.dtype).cpu()):
            raise ValueError("MTP conditioning requires the Target's own frozen embedding")
        self.mtp_source.validate_native_weights(tensors)

    # -- parameter policy -------------------------------------------------------
    def freeze_embedding(self) -> None:
        self.embed_tokens.weight.requires_grad_(False)

    def load_embedding(self, weight: torch.Tensor) -> None:
        with torch.no_grad():
            self.embed_tokens.weight.copy_(weight.to(self.embed_tokens.weight))
        self.freeze_embedding()

    # -- pieces of the forward --------------------------------------------------
    def extract_context_feature(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """``[T, K*Dt]`` concatenated captured layers -> ``[T, D]``."""
        if self.fc_norm is not None:
            dt = self.config.target_hidden_size
            parts = hidden_states.split(dt, dim=-1)
            hidden_states = torch.cat([n(p) for n, p in zip(self.fc_norm, parts)], -1)
        return self.context_norm(self.context_proj(hidden_states))

    def forward(self, context_feature: torch.Tensor, draft_embeds: torch.Tensor,
                context_positions: torch.Tensor, draft_positions: torch.Tensor,
                intervals, aux: Optional[dict] = None) -> torch.Tensor:
        """``intervals`` is one ``[Q, 4]`` table or a list with one table per layer."""
        x = draft_embeds
        kv_pos = torch.cat([context_positions, draft_positions])
        for i, layer in enumerate(self.layers):
            iv = intervals[i] if isinstance(intervals, (list, tuple)) else intervals
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(layer, x, context_feature, draft_positions, kv_pos, iv, aux,
                               use_reentrant=False)
            else:
                x = layer(x, context_feature, draft_positions, kv_pos, iv, aux)
        return self.final_norm(x)
