"""Compressed sparse attention (CSA) for DFlash-family drafts: an overlapping ratio-``m`` compressor turns the
context into one key/value entry per token group, a Lightning indexer ranks the groups, and each query attends
raw sliding-window tokens + its own block + compressed entries.

Behaviour (reference: aspec/models/draft/csa.py:374-528 compressor, :796-855,1160-1193 indexer and KL,
:1717-1803 attention over raw window ∪ block ∪ compressed entries, :1805-1984 layer):

* compressor: two fp32 projections per token (``kv_proj``, ``gate_proj`` -> 2 series); group ``g`` pools series 0 of
  group ``g-1`` (same document only) and series 1 of group ``g`` with a softmax gate over the ``2m`` entries plus a
  learned per-slot bias, then RMSNorm; the value is the pooled vector, the key its RoPE rotation at the group's
  position;
* eligible groups: same document, ending at or before the anchor;
* indexer (inputs detached): its own 1-head compressor for keys, ``q_proj`` + RoPE, score
  ``= sum_h relu(q_h . k_g) * w_h``, ``w = weights_proj(x) * di^-1/2 * Hi^-1/2``;
* ``dense``: all eligible groups; ``indexer_warmup``: KL(head-summed main softmax over eligible compressed keys ||
  softmax(score)), main model frozen; ``sparse``: top ``index_topk`` groups, KL on the selected set.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from aspec_b200.models.draft.dflash import DFlashAttention
from aspec_b200.models.draft.sparse_common import (build_group_layout, eligible_groups, indexed_attention, kl_rows,
                                                   masked_log_softmax, own_block_index, rotary)
from aspec_b200.ops.fused_params import fused_linear
from aspec_b200.ops.norm import RMSNorm
from aspec_b200.ops.rope import qk_norm_rope


class CSAOverlappingCompressor(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, ratio: int, rope_theta: float, eps: float):
        super().__init__()
        self.num_heads, self.head_dim, self.ratio, self.rope_theta = num_heads, head_dim, ratio, rope_theta
        width = num_heads * head_dim
        self.kv_proj = nn.Linear(hidden_size, 2 * width, bias=False)
        self.gate_proj = nn.Linear(hidden_size, 2 * width, bias=False)
        self.position_bias = nn.Parameter(torch.zeros(ratio, 2 * width, dtype=torch.float32))
        self.norm = RMSNorm(head_dim, eps=eps)
        self.keep_projection_fp32()

    def keep_projection_fp32(self) -> None:
        """The gate's softmax is sensitive to bf16 rounding; these weights stay fp32 through dtype casts."""
        self.kv_proj.float()
        self.gate_proj.float()
        self.position_bias.data = self.position_bias.data.float()

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        self.keep_projection_fp32()
        return out

    def forward(self, ctx: torch.Tensor, layout):
        """``ctx [T, D]`` -> ``(value [G, H, d], key [G, H, d])``."""
        G, m, H, d = layout.num_groups, self.ratio, self.num_heads, self.head_dim
        if G == 0:
            zero = (ctx.reshape(-1)[:0].sum() + sum(p.reshape(-1)[:0].sum() for p in self.parameters())).to(ctx.dtype)
            empty = ctx.new_zeros(0, H, d) + zero
            return empty, empty
        rows = ctx.float()[layout.token_index.reshape(-1)]
        vals = self.kv_proj(rows).view(G, m, 2, H, d)
        gates = (self.gate_proj(rows).view(G, m, -1) + self.position_bias[None]).view(G, m, 2, H, d)
        prev_v = torch.roll(vals[:, :, 0], 1, 0)
        prev_g = torch.roll(gates[:, :, 0], 1, 0).masked_fill(layout.first[:, None, None, None], float("-inf"))
        v = torch.cat([prev_v, vals[:, :, 1]], 1)
        g = torch.cat([prev_g, gates[:, :, 1]], 1)
        pooled = self.norm((v * g.softmax(1)).sum(1).to(ctx.dtype))
        return pooled, rotary(pooled, layout.position, d, self.rope_theta)


class CSALightningIndexer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.num_heads, self.head_dim, self.topk = config.index_n_heads, config.index_head_dim, config.index_topk
        self.rope_theta = config.compress_rope_theta
        self.key_compressor = CSAOverlappingCompressor(config.hidden_size, 1, self.head_dim,
                                                       config.compress_ratios[layer_idx], self.rope_theta,
                                                       config.rms_norm_eps)
        self.q_proj = nn.Linear(config.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.weights_proj = nn.Linear(config.hidden_size, self.num_heads, bias=False)
        self.scale = self.head_dim ** -0.5 * self.num_heads ** -0.5

    def forward(self, x, ctx, q_pos, layout):
        x, ctx = x.detach(), ctx.detach()
        _, key = self.key_compressor(ctx, layout)
        q = self.q_proj(x.to(self.q_proj.weight.dtype)).view(x.shape[0], self.num_heads, self.head_dim)
        q = rotary(q, q_pos, self.head_dim, self.rope_theta)
        w = self.weights_proj(x.to(self.weights_proj.weight.dtype)).float() * self.scale
        return (torch.einsum("nhd,gd->nhg", q.float(), key[:, 0].float()).relu_() * w[:, :, None]).sum(1)


class CSAAttention(DFlashAttention):
    def __init__(self, config, layer_idx: int):
        super().__init__(config, layer_idx)
        self.stage = config.csa_training_stage
        self.ratio = config.compress_ratios[layer_idx]
        self.workspace_bytes = config.csa_workspace_bytes
        self.compressor = CSAOverlappingCompressor(config.hidden_size, self.num_kv_heads, self.head_dim, self.ratio,
                                                   config.compress_rope_theta, config.rms_norm_eps)
        self.indexer = CSALightningIndexer(config, layer_idx)
        self.compute_auxiliary_loss = True

    def _teacher(self, q, ckey, mask):
        """Head-summed softmax of the main queries over the (masked) compressed keys, renormalised."""
        g = self.num_heads // self.num_kv_heads
        s = torch.einsum("nhd,ghd->nhg", q.float(), ckey.repeat_interleave(g, 1).float()) * self.scale
        logp, valid = masked_log_softmax(s.reshape(-1, s.shape[-1]), mask[:, None].expand_as(s).reshape(-1, s.shape[-1]))
        p = (logp.exp().view_as(s) * mask[:, None]).sum(1)
        return p / p.sum(-1, keepdim=True).clamp_min(1e-12)

    def forward(self, x, ctx, q_pos, kv_pos, intervals, aux=None, attn_override=None):
        Q, T = x.shape[0], ctx.shape[0]
        d, hk = self.head_dim, self.num_kv_heads
        frozen = self.stage == "indexer_warmup"
        aux = aux if aux is not None else {}
        doc_lo = aux.get("query_doc_start", intervals[:, 0]).long()
        anchor = aux.get("query_anchor", intervals[:, 1]).long()
        layout = build_group_layout(doc_lo, anchor, kv_pos[:T], self.ratio)
        with torch.set_grad_enabled(torch.is_grad_enabled() and not frozen):
            q = self.q_proj(x).view(Q, self.num_heads, d)
            kv = fused_linear(torch.cat([ctx, x], 0), [self.k_proj.weight, self.v_proj.weight])
            k = kv[:, : hk * d].reshape(T + Q, hk, d)
            v = kv[:, hk * d:].reshape(T + Q, hk, d)
            inv = self.rope_freqs.get(x.device)
            q = qk_norm_rope(q, self.q_norm.weight, q_pos, inv, self.eps, self.rope_scaling)
            k = qk_norm_rope(k, self.k_norm.weight, kv_pos, inv, self.eps, self.rope_scaling)
            cval, ckey = self.compressor(ctx, layout)
        elig = eligible_groups(layout, doc_lo, anchor)
        G = layout.num_groups
        visible = elig
        if self.stage != "dense" and (self.compute_auxiliary_loss or self.stage == "sparse"):
            score = self.indexer(x, ctx, q_pos, layout)
            if self.stage == "indexer_warmup":
                with torch.no_grad():
                    target = self._teacher(q.detach(), ckey.detach(), elig)
                logp, valid = masked_log_softmax(score, elig)
                loss = kl_rows(target, logp, valid)
            else:
                topk = min(self.indexer.topk, G)
                with torch.no_grad():
                    top = score.detach().masked_fill(~elig, float("-inf")).topk(topk, -1)
                    sel, sel_ok = top.indices, torch.isfinite(top.values)
                    visible = torch.zeros_like(elig).scatter_(1, sel, sel_ok)
                    target = self._teacher(q.detach(), ckey.detach(), visible).gather(1, sel)
                logp, valid = masked_log_softmax(score.gather(1, sel), sel_ok)
                loss = kl_rows(target, logp, valid)
            if self.compute_auxiliary_loss:
                aux.setdefault("csa_losses", []).append(loss)
        with torch.set_grad_enabled(torch.is_grad_enabled() and not frozen):
            out = self._attend(q, k, v, ckey, cval, visible, intervals, T)
        return self.o_proj(out.reshape(Q, -1))

    def _attend(self, q, k, v, ckey, cval, visible, intervals, T):
        """Raw window tokens ∪ own block ∪ visible compressed entries, chunked over queries."""
        Q, G = q.shape[0], ckey.shape[0]
        lo, hi = intervals[:, 0].long(), intervals[:, 1].long()
        width = int((hi - lo).max().item()) if Q else 0
        blk, blk_ok = own_block_index(intervals, k.shape[0])
        keys = torch.cat([k, ckey.to(k.dtype)], 0)
        vals = torch.cat([v, cval.to(v.dtype)], 0)
        per_row = (width + blk.shape[1] + G) * self.num_kv_heads * self.head_dim * 2 * 4
        rows = max(int(self.workspace_bytes // max(per_row, 1)), 1)
        from aspec_b200.ops.sparse_attention import _kernel_ok
        if _kernel_ok(q, keys, vals):
            rows = max(Q, 1)            # the kernel gathers tile by tile: no per-row workspace to bound
        comp = (k.shape[0] + torch.arange(G, device=q.device))[None]
        outs = []
        for s0 in range(0, Q, rows):
            sl = slice(s0, min(s0 + rows, Q))
            raw = lo[sl, None] + torch.arange(width, device=q.device)[None]
            raw_ok = raw < hi[sl, None]
            idx = torch.cat([raw.clamp(max=T - 1), blk[sl], comp.expand(raw.shape[0], -1)], 1)
            ok = torch.cat([raw_ok, blk_ok[sl], visible[sl]], 1)
            outs.append(indexed_attention(q[sl], keys, vals, idx, ok, self.scale))
        return torch.cat(outs, 0) if outs else q.new_zeros(q.shape)

    def trainable_parameter_names(self):
        return [n for n, _ in self.named_parameters() if n.startswith("indexer.")] if self.stage == "indexer_warmup" else None
