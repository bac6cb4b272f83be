"""EAGLE3 draft: one decoder layer ("midlayer") fed ``cat(norm(embed), norm(hidden))``, own LM head.

Architecture (reference: aspec/models/draft/llama3_eagle.py:2331-2484): ``fc: Linear(K * Dt -> D)`` turns the
captured Target layers into the depth-0 hidden state; the attention input is the concatenation of the
normalised token embedding and the normalised hidden state (width ``2D``); the MLP follows
``post_attention_layernorm``; ``norm`` + ``lm_head`` (optionally over a pruned draft vocabulary with
``t2d`` / ``d2t``) produce logits.

The test-time-training recurrence is expressed over packed tokens with the interval attention kernel:
keys of depth 0 are laid out first (``T`` rows, causal inside each document) and the keys of the later
depths are stored token-major right after them, so that the "one diagonal key per earlier depth" of
query ``t`` (aspec/models/draft/llama3_eagle.py:1229-1263) is the contiguous range
``[T + t * (L - 1), T + t * (L - 1) + depth)`` - exactly the kernel's second interval.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from aspec_b200.config.draft_config import Eagle3Config
from aspec_b200.config.rope import mrope_axis_of_frequency, rope_inverse_frequencies
from aspec_b200.models.draft.base import Eagle3DraftModel
from aspec_b200.models.draft.dflash import DFlashMLP, _Weight
from aspec_b200.ops.attention import interval_attention
from aspec_b200.ops.fused_params import allocate_adjacent, fused_linear
from aspec_b200.ops.linear import Linear
from aspec_b200.ops.norm import RMSNorm
from aspec_b200.ops.rope import RopeFrequencies, qk_norm_rope


class EagleAttention(nn.Module):
    def __init__(self, config, input_width: Optional[int] = None, use_rope: bool = True, window: Optional[int] = None):
        super().__init__()
        D, d = config.hidden_size, config.head_dim
        width = input_width or 2 * D
        self.use_rope, self.window = use_rope, window
        self.num_heads, self.num_kv_heads, self.head_dim = config.num_attention_heads, config.num_key_value_heads, d
        qw, kw, vw = allocate_adjacent([(self.num_heads * d, width), (self.num_kv_heads * d, width),
                                        (self.num_kv_heads * d, width)])
        for w in (qw, kw, vw):
            nn.init.normal_(w, std=0.02)
        self.q_proj, self.k_proj, self.v_proj = _Weight(qw), _Weight(kw), _Weight(vw)
        self.o_proj = Linear(self.num_heads * d, D)
        params = {"rope_type": "default", "rope_theta": float(config.rope_theta)}
        scaling = getattr(config, "rope_scaling", None)
        if scaling:
            params.update(scaling)
            params["rope_type"] = scaling.get("rope_type", scaling.get("type", "default"))
            params.setdefault("original_max_position_embeddings", config.max_position_embeddings)
        inv, self.rope_scaling = rope_inverse_frequencies(d, params)
        self.rope_freqs = RopeFrequencies(inv)
        # multi-axis RoPE: the stream (temporal / height / width) that rotates each frequency; used when a row brings
        # three position streams, which only rows with image or video spans do
        self.mrope_axes = (RopeFrequencies(mrope_axis_of_frequency(d, scaling["mrope_section"]))
                           if scaling and params["rope_type"] == "mrope" else None)
        self.scale = d ** -0.5

    def project(self, x: torch.Tensor, positions: torch.Tensor):
        """``x [T, 2D]`` -> rotated ``q [T, Hq, d]``, ``k [T, Hkv, d]`` and ``v [T, Hkv, d]``."""
        T = x.shape[0]
        hq, hk, d = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = fused_linear(x, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight])
        q = qkv[:, : hq * d].reshape(T, hq, d)
        k = qkv[:, hq * d:(hq + hk) * d].reshape(T, hk, d)
        v = qkv[:, (hq + hk) * d:].reshape(T, hk, d)
        if self.use_rope:
            inv = self.rope_freqs.get(x.device)
            axes = self.mrope_axes.get(x.device) if self.mrope_axes is not None and positions.dim() == 2 else None
            q = qk_norm_rope(q, None, positions, inv, 0.0, self.rope_scaling, axes)
            k = qk_norm_rope(k, None, positions, inv, 0.0, self.rope_scaling, axes)
        return q, k.contiguous(), v.contiguous()


class EagleDecoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self_attn = EagleAttention(config)
        self.mlp = DFlashMLP(config.hidden_size, config.intermediate_size)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.hidden_norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def attention_input(self, embeds: torch.Tensor, hidden: torch.Tensor):
        """``(attention input, residual stream)`` of one TTT depth."""
        return torch.cat([self.input_layernorm(embeds), self.hidden_norm(hidden)], -1), hidden


class LlamaForCausalLMEagle3(Eagle3DraftModel):
    config_class = Eagle3Config
    decoder_layer_class = EagleDecoderLayer

    def __init__(self, config):
        super().__init__()
        self.config = config
        D, Dt = config.hidden_size, config.target_hidden_size
        self.num_aux = int(config.num_aux_hidden_states)
        self.fc = Linear(self.num_aux * Dt, D)
        self.fc_norm = (nn.ModuleList([RMSNorm(Dt, eps=config.rms_norm_eps) for _ in range(self.num_aux)])
                        if getattr(config, "fc_norm", False) else None)
        self.embed_tokens = nn.Embedding(config.vocab_size, D)
        self.embed_tokens.weight.requires_grad_(False)
        self.midlayer = self.decoder_layer_class(config)
        self.norm = RMSNorm(D, eps=config.rms_norm_eps)
        self.lm_head = Linear(D, config.draft_vocab_size)
        self.init_vocab_buffers(config.vocab_size, config.draft_vocab_size)
        self.norm_output = bool(getattr(config, "norm_output", False))
        self.gradient_checkpointing = False

    # -- pieces used by the training wrapper -------------------------------------------------------
    def project_hidden_states(self, features: torch.Tensor) -> torch.Tensor:
        if self.fc_norm is not None:
            parts = features.split(self.config.target_hidden_size, dim=-1)
            features = torch.cat([n(p) for n, p in zip(self.fc_norm, parts)], -1)
        return self.fc(features)

    def embed_input_ids(self, ids: torch.Tensor) -> torch.Tensor:
        return self.embed_tokens(ids.clamp(0, self.config.vocab_size - 1))

    def backbone(self, embeds: torch.Tensor, hidden: torch.Tensor, positions: torch.Tensor, depth: int,
                 cache: Optional[Tuple[torch.Tensor, torch.Tensor, List, List]], doc_start: torch.Tensor,
                 ttt_length: int):
        """One TTT depth over ``T`` packed tokens.  Returns the new hidden state and the extended cache."""
        layer = self.midlayer
        x, residual = layer.attention_input(embeds, hidden)
        ex = getattr(self, "ulysses", None)
        if ex is not None:
            # Sequence parallel: ``embeds`` / ``hidden`` are this rank's rows, ``positions`` / ``doc_start`` describe ALL
            # rows of the packed sequence; the exchange moves QKV to head owners and attention outputs back.
            attn_out, cache = self._ulysses_attention(layer, x, positions, depth, cache, doc_start, ttt_length, ex)
            h = residual + attn_out
        else:
            q, k, v = layer.self_attn.project(x, positions + depth)
            o, cache = self._attend(layer.self_attn, q, k, v, depth, cache, doc_start, ttt_length)
            h = residual + layer.self_attn.o_proj(o.reshape(o.shape[0], -1))
        h = h + self._mlp(layer, layer.post_attention_layernorm(h), depth)
        return h, cache

    @staticmethod
    def _attend(attn, q, k, v, depth: int, cache, doc_start: torch.Tensor, ttt_length: int):
        """Attention of one TTT depth over ``T`` rows: causal keys of depth 0 plus the row's own keys of depths
        ``1..depth``.  Returns the output ``[T, H, d]`` and the extended cache ``(k0, v0, [k_1..], [v_1..])``."""
        T = q.shape[0]
        L1 = max(ttt_length - 1, 1)
        t = torch.arange(T, device=q.device)
        if depth == 0:
            k0, v0, dk, dv = k, v, [], []
        else:
            k0, v0, dk, dv = cache
            dk, dv = dk + [k], dv + [v]
        if dk:
            n_pad = L1 - len(dk)
            k_all = torch.cat([k0, torch.stack(dk + [torch.zeros_like(k)] * n_pad, 1).reshape(T * L1, *k.shape[1:])])
            v_all = torch.cat([v0, torch.stack(dv + [torch.zeros_like(v)] * n_pad, 1).reshape(T * L1, *v.shape[1:])])
        else:
            k_all, v_all = k0, v0
        window = getattr(attn, "window", None)
        lo = doc_start if window is None else torch.maximum(doc_start, t + 1 - window)
        intervals = torch.stack([lo, t + 1, T + t * L1, T + t * L1 + depth], -1).to(torch.int32)
        o, _ = interval_attention(q, k_all, v_all, intervals, attn.scale)
        return o, (k0, v0, dk, dv)

    @staticmethod
    def _attend_ring(attn, q, k, v, depth: int, cache, doc_start: torch.Tensor, ttt_length: int, row0: int, ring_group):
        """``_attend`` when the rows are one shard of a sequence spread over a ring: the causal depth-0 keys live on every
        rank of the ring (``parallel.ring_attention``), the keys of depths ``1..depth`` are each row's own and stay local.
        ``doc_start`` holds GLOBAL row indices, ``row0`` is the global index of this shard's first row."""
        from aspec_b200.parallel.ring_attention import ring_attention
        S = q.shape[0]
        L1 = max(ttt_length - 1, 1)
        t = torch.arange(S, device=q.device)
        if depth == 0:
            k0, v0, dk, dv = k, v, [], []
        else:
            k0, v0, dk, dv = cache
            dk, dv = dk + [k], dv + [v]
        n_pad = L1 - len(dk)
        k_all = torch.cat([k0, torch.stack(dk + [torch.zeros_like(k)] * n_pad, 1).reshape(S * L1, *k.shape[1:])])
        v_all = torch.cat([v0, torch.stack(dv + [torch.zeros_like(v)] * n_pad, 1).reshape(S * L1, *v.shape[1:])])
        tg = t + row0
        window = getattr(attn, "window", None)
        lo = doc_start if window is None else torch.maximum(doc_start, tg + 1 - window)
        intervals = torch.stack([lo, tg + 1, S + t * L1, S + t * L1 + depth], -1).to(torch.int32)
        o, _ = ring_attention(q, k_all, v_all, intervals, S, attn.scale, ring_group)
        return o, (k0, v0, dk, dv)

    def _ulysses_attention(self, layer, x, positions_all, depth: int, cache, doc_start_all, ttt_length: int, ex):
        from aspec_b200.parallel.ulysses import group_qkv_rows
        from aspec_b200.parallel.ulysses_attention import ulysses_block
        sa = layer.self_attn
        p = ex.world
        if sa.num_heads % p or sa.num_kv_heads % p:
            raise ValueError("attention head counts must be divisible by the sequence-parallel size")
        hq, hk, d = sa.num_heads // p, sa.num_kv_heads // p, sa.head_dim
        w_grouped = group_qkv_rows(sa.q_proj.weight, sa.k_proj.weight, sa.v_proj.weight, p, d)
        state = {}

        ring = getattr(self, "ring", None)          # (ring index, ring size, process group): Ulysses x ring

        def core(qkv: torch.Tensor) -> torch.Tensor:            # the exchange group's rows, this rank's heads
            T = qkv.shape[0]
            q = qkv[:, : hq * d].reshape(T, hq, d)
            k = qkv[:, hq * d:(hq + hk) * d].reshape(T, hk, d)
            v = qkv[:, (hq + hk) * d:].reshape(T, hk, d)
            # with a ring stage the exchange group holds one contiguous shard of the packed sequence
            row0 = ring[0] * T if ring is not None else 0
            pos = positions_all[row0:row0 + T] + depth
            starts = doc_start_all[row0:row0 + T]
            if sa.use_rope:
                inv = sa.rope_freqs.get(qkv.device)          # text rows: one position stream, also under mrope
                q = qk_norm_rope(q.contiguous(), None, pos, inv, 0.0, sa.rope_scaling)
                k = qk_norm_rope(k.contiguous(), None, pos, inv, 0.0, sa.rope_scaling)
            if ring is not None and ring[1] > 1:
                o, state["cache"] = self._attend_ring(sa, q, k.contiguous(), v.contiguous(), depth, cache, starts, ttt_length,
                                                      row0, ring[2])
            else:
                o, state["cache"] = self._attend(sa, q, k.contiguous(), v.contiguous(), depth, cache, starts, ttt_length)
            return o.reshape(T, hq * d)

        ex.set_rows(x.shape[0])
        out = ulysses_block(x, w_grouped, sa.o_proj.weight, ex, core)
        return out, state["cache"]

    def _mlp(self, layer, x: torch.Tensor, depth: int) -> torch.Tensor:
        return layer.mlp(x)

    def next_depth_hidden(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.norm(hidden) if self.norm_output else hidden

    def get_lm_head_params(self):
        return self.norm.weight, self.lm_head.weight, self.norm.eps

    def get_lm_head_up_weight(self):
        return None

    def commit_router_load(self) -> None:
        pass
