"""Materialised multi-head latent attention (MLA) for DFlash-family drafts and the DeepSeek EAGLE draft.

Queries go through an optional low-rank bottleneck (``q_a_proj -> RMSNorm -> q_b_proj``); keys and values come
from a shared latent (``kv_a_proj_with_mqa -> RMSNorm -> kv_b_proj``) plus one rotary key shared by all heads.
The latent is expanded before attention ("materialised"), so the layout is MHA with
``qk_nope + qk_rope`` query/key width and a separate value width
(reference: aspec/models/draft/dspark.py:176-484, aspec/models/draft/deepseek_eagle.py:89-575,
aspec/config/draft_attention.py:21-67).  The (192, 128) head shape of the shipped MLA configurations runs the
interval attention kernels (their 192-wide query/key instantiation); other widths take the bounded fp32 statement.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from aspec_b200.ops.attention import interval_attention
from aspec_b200.ops.linear import Linear
from aspec_b200.ops.norm import RMSNorm
from aspec_b200.ops.rope import RopeFrequencies, qk_norm_rope_reference


class MLAAttention(nn.Module):
    def __init__(self, config, layer_idx: int = 0, input_width: int = None):
        super().__init__()
        D = config.hidden_size
        width = input_width or D
        self.num_heads = config.num_attention_heads
        self.nope, self.rope, self.v_dim = config.qk_nope_head_dim, config.qk_rope_head_dim, config.v_head_dim
        self.q_head_dim = self.nope + self.rope
        self.kv_lora_rank = config.kv_lora_rank
        q_rank = getattr(config, "q_lora_rank", None)
        if q_rank:
            self.q_a_proj = Linear(width, q_rank)
            self.q_a_layernorm = RMSNorm(q_rank, eps=config.rms_norm_eps)
            self.q_b_proj = Linear(q_rank, self.num_heads * self.q_head_dim)
            self.q_proj = None
        else:
            self.q_proj = Linear(width, self.num_heads * self.q_head_dim)
        self.kv_a_proj_with_mqa = Linear(width, self.kv_lora_rank + self.rope)
        self.kv_a_layernorm = RMSNorm(self.kv_lora_rank, eps=config.rms_norm_eps)
        self.kv_b_proj = Linear(self.kv_lora_rank, self.num_heads * (self.nope + self.v_dim))
        self.o_proj = Linear(self.num_heads * self.v_dim, D)
        self.rope_freqs = RopeFrequencies([float(config.rope_theta) ** (-(2.0 * i) / self.rope) for i in range(self.rope // 2)])
        self.scale = self.q_head_dim ** -0.5

    def queries(self, x, positions):
        q = self.q_proj(x) if self.q_proj is not None else self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x)))
        q = q.view(x.shape[0], self.num_heads, self.q_head_dim)
        q_rot = qk_norm_rope_reference(q[..., self.nope:], None, positions, self.rope_freqs.get(x.device), 0.0)
        return torch.cat([q[..., : self.nope], q_rot], -1)

    def keys_values(self, x, positions):
        n = x.shape[0]
        a = self.kv_a_proj_with_mqa(x)
        latent, k_rope = a[:, : self.kv_lora_rank], a[:, self.kv_lora_rank:]
        kv = self.kv_b_proj(self.kv_a_layernorm(latent)).view(n, self.num_heads, self.nope + self.v_dim)
        k_rope = qk_norm_rope_reference(k_rope[:, None], None, positions, self.rope_freqs.get(x.device), 0.0)
        k = torch.cat([kv[..., : self.nope], k_rope.expand(-1, self.num_heads, -1)], -1)
        return k, kv[..., self.nope:]

    def forward(self, x, ctx, q_pos, kv_pos, intervals, aux=None):
        q = self.queries(x, q_pos)
        k, v = self.keys_values(torch.cat([ctx, x], 0), kv_pos)
        o, _ = interval_attention(q, k.contiguous(), v.contiguous(), intervals, self.scale)
        return self.o_proj(o.reshape(x.shape[0], -1))
