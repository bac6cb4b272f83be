"""Qwen-style sparse attention (QSA) for DFlash-family drafts: an MQA indexer over mean-pooled key groups
picks, once per draft block, the groups whose raw tokens the block attends.

Behaviour (reference: aspec/models/draft/qsa.py:350-423,910-1189,1276-1437,1440-1525):

* indexer (inputs NOT detached): ``q = rope(RMSNorm(q_proj(x)))`` -> ``[Hi, di]`` per block (the block's first
  query row represents it), keys = mean of ``k_proj(ctx)`` over groups of ``ratio`` tokens, RMSNorm, partial
  RoPE at the group's first position; score ``= sum_h relu(q_h . k_g) * di^-1/2``;
* eligible groups are complete, in the query's document and end at or before the anchor; the ragged
  ``< ratio`` tail before the anchor is always attended;
* ``indexer_warmup``: teacher = head-summed main-attention softmax over visible context + own block,
  max-pooled per group, renormalised over eligible groups; loss = KL(teacher || softmax(score));
* ``sparse``: top ``token_budget / ratio`` groups per block; KL on the selected set; attention over the selected
  groups' raw tokens + tail + own block.  The per-block KL is repeated for every row of the block.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from aspec_b200.models.draft.dflash import DFlashAttention
from aspec_b200.models.draft.sparse_common import (build_group_layout, eligible_groups, indexed_attention, kl_rows,
                                                   masked_log_softmax, own_block_index, rotary)
from aspec_b200.ops.attention import interval_attention
from aspec_b200.ops.fused_params import fused_linear
from aspec_b200.ops.linear import Linear
from aspec_b200.ops.norm import RMSNorm
from aspec_b200.ops.rope import qk_norm_rope


class QSAIndexer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_heads, self.head_dim = config.qsa_index_n_heads, config.qsa_index_head_dim
        self.ratio, self.token_budget = config.qsa_compress_ratio, config.qsa_token_budget
        self.block_topk = self.token_budget // self.ratio
        self.workspace_bytes = config.qsa_workspace_bytes
        self.rope_dim, self.rope_theta = config.qsa_rope_dim, config.qsa_rope_theta
        self.q_proj = Linear(config.hidden_size, self.num_heads * self.head_dim)
        self.k_proj = Linear(config.hidden_size, self.head_dim)
        self.q_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.k_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.scale = self.head_dim ** -0.5

    def project(self, x, ctx, q_pos, layout):
        q = self.q_norm(self.q_proj(x).view(x.shape[0], self.num_heads, self.head_dim))
        q = rotary(q, q_pos, self.rope_dim, self.rope_theta)
        tk = self.k_proj(ctx)
        pooled = tk[layout.token_index].float().mean(1).to(tk.dtype)
        k = rotary(self.k_norm(pooled)[:, None], layout.position, self.rope_dim, self.rope_theta)[:, 0]
        return q, k

    def scores(self, q, k):
        return torch.einsum("nhd,gd->nhg", q.float(), k.float()).relu_().sum(1) * self.scale


class QSAAttention(DFlashAttention):
    def __init__(self, config, layer_idx: int):
        super().__init__(config, layer_idx)
        self.stage = config.qsa_training_stage
        self.indexer = QSAIndexer(config)
        self.compute_auxiliary_loss = True
        self.block_size = int(getattr(config, "block_size", 0) or 0)

    def _token_teacher(self, q, k, iv, T):
        """Head-summed softmax over visible context + own block; returns the context part ``[n, T]``."""
        lo, hi = iv[:, 0].long(), iv[:, 1].long()
        g = self.num_heads // self.num_kv_heads
        t = torch.arange(T, device=q.device)[None]
        vis = (t >= lo[:, None]) & (t < hi[:, None])
        blk, blk_ok = own_block_index(iv, k.shape[0])
        s_ctx = torch.einsum("nhd,thd->nht", q.float(), k[:T].repeat_interleave(g, 1).float()) * self.scale
        s_blk = torch.einsum("nhd,nshd->nhs", q.float(), k[blk].repeat_interleave(g, 2).float()) * self.scale
        s = torch.cat([s_ctx.masked_fill(~vis[:, None], float("-inf")),
                       s_blk.masked_fill(~blk_ok[:, None], float("-inf"))], -1)
        p = torch.softmax(s, -1)[..., :T]
        return torch.where(vis[:, None], p, torch.zeros_like(p)).sum(1)

    def forward(self, x, ctx, q_pos, kv_pos, intervals, aux=None, attn_override=None):
        if self.stage == "dense":
            return super().forward(x, ctx, q_pos, kv_pos, intervals, aux=aux, attn_override=attn_override)
        Q, T = x.shape[0], ctx.shape[0]
        d, hk = self.head_dim, self.num_kv_heads
        frozen = self.stage == "indexer_warmup"
        with torch.set_grad_enabled(torch.is_grad_enabled() and not frozen):
            q = self.q_proj(x).view(Q, self.num_heads, d)
            kv = fused_linear(torch.cat([ctx, x], 0), [self.k_proj.weight, self.v_proj.weight])
            k = kv[:, : hk * d].reshape(T + Q, hk, d)
            v = kv[:, hk * d:].reshape(T + Q, hk, d)
            inv = self.rope_freqs.get(x.device)
            q = qk_norm_rope(q, self.q_norm.weight, q_pos, inv, self.eps, self.rope_scaling)
            k = qk_norm_rope(k, self.k_norm.weight, kv_pos, inv, self.eps, self.rope_scaling)
        lo, hi = intervals[:, 0].long(), intervals[:, 1].long()
        block = int((aux or {}).get("block_size", self.block_size))
        if Q % block:
            raise ValueError("QSA draft queries must contain one complete block per anchor")
        rep = torch.arange(0, Q, block, device=x.device)
        layout = build_group_layout(lo, hi, kv_pos[:T], self.indexer.ratio)
        G = layout.num_groups
        xi, ci = (x.detach(), ctx.detach()) if frozen else (x, ctx)
        iq, ik = self.indexer.project(xi[rep], ci, q_pos[rep], layout)
        rows = max(int(self.indexer.workspace_bytes // max((T + block) * 4 * (self.num_heads + 2), 1)), 1)
        losses, picks = [], []
        topk = min(self.indexer.block_topk, G)
        for s0 in range(0, rep.numel(), rows):
            r = rep[s0: s0 + rows]
            elig = eligible_groups(layout, lo[r], hi[r])
            score = self.indexer.scores(iq[s0: s0 + rows], ik)
            with torch.no_grad():
                tok = self._token_teacher(q[r].detach(), k.detach(), intervals[r], T)
                pooled = tok[:, layout.token_index.reshape(-1)].view(r.numel(), G, -1).amax(-1) if G else tok[:, :0]
            if self.stage == "indexer_warmup":
                target = pooled * elig
                target = target / target.sum(-1, keepdim=True).clamp_min(1e-12)
                logp, valid = masked_log_softmax(score, elig)
                losses.append(kl_rows(target, logp, valid))
                continue
            with torch.no_grad():
                top = score.detach().masked_fill(~elig, float("-inf")).topk(topk, -1) if topk else None
                sel = top.indices if topk else score.new_zeros((r.numel(), 0), dtype=torch.long)
                sel_ok = torch.isfinite(top.values) if topk else sel.bool()
            picks.append((sel, sel_ok))
            target = pooled.gather(1, sel) * sel_ok
            target = target / target.sum(-1, keepdim=True).clamp_min(1e-12)
            logp, valid = masked_log_softmax(score.gather(1, sel), sel_ok)
            losses.append(kl_rows(target, logp, valid))
        if aux is not None and self.compute_auxiliary_loss and losses:
            aux.setdefault("qsa_losses", []).append(torch.cat(losses).repeat_interleave(block))
        if frozen:
            with torch.no_grad():
                o, _ = interval_attention(q, k, v, intervals, self.scale)
            return self.o_proj(o.reshape(Q, -1))
        sel = torch.cat([p[0] for p in picks]); sel_ok = torch.cat([p[1] for p in picks])
        return self.o_proj(self._sparse_core(q, k, v, sel, sel_ok, layout, intervals, rep, block, T).reshape(Q, -1))

    def _sparse_core(self, q, k, v, sel, sel_ok, layout, intervals, rep, block, T):
        """One gather per block: selected groups' raw tokens + ragged tail + the block itself."""
        r = layout.ratio
        lo, hi = intervals[rep, 0].long(), intervals[rep, 1].long()
        nb = rep.numel()
        tok = layout.token_index[sel.clamp_min(0)].reshape(nb, -1) if sel.shape[1] else sel
        tok_ok = sel_ok.repeat_interleave(r, 1) if sel.shape[1] else sel_ok
        tail0 = hi - (hi - lo).remainder(r)
        tail = tail0[:, None] + torch.arange(r - 1, device=q.device)[None]
        tail_ok = tail < hi[:, None]
        blk, blk_ok = own_block_index(intervals, k.shape[0])
        idx = torch.cat([torch.cat([tok, tail.clamp(max=T - 1)], 1).repeat_interleave(block, 0), blk], 1)
        ok = torch.cat([torch.cat([tok_ok, tail_ok], 1).repeat_interleave(block, 0), blk_ok], 1)
        return indexed_attention(q, k, v, idx, ok, self.scale)

    def trainable_parameter_names(self):
        return [n for n, _ in self.named_parameters() if n.startswith("indexer.")] if self.stage == "indexer_warmup" else None
