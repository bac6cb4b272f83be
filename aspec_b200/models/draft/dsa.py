"""DeepSeek-style sparse attention (DSA) for DFlash-family drafts: a per-query token indexer plus
attention over the selected context tokens, trained in three stages.

Behaviour (reference: aspec/models/draft/dsa.py:51-451):

* indexer (inputs detached): ``q = q_b(RMSNorm(q_a(x)))`` -> ``[Q, Hi, di]``, ``k = LayerNorm(k_proj(ctx))`` ->
  ``[T, di]``, rotate-half RoPE on the first ``rope_dim`` dims, score ``= sum_h relu(q_h . k) * w_h`` with
  ``w = weights_proj(x) * di^-1/2 * Hi^-1/2``;
* ``dense``: ordinary attention, indexer untouched;
* ``indexer_warmup``: the main attention's head-summed softmax over the eligible context (strictly before
  the anchor, same document) is the teacher; loss = KL(teacher || softmax(score)); only the indexer trains;
* ``sparse``: without gradient each query keeps its top-``token_budget`` context tokens, the KL is taken on
  that set, and attention runs over the selected tokens plus the query's own block.

Eligibility is read from the interval table (first interval = visible context).  Work is chunked over
queries so that no ``[Q, T]`` fp32 tensor larger than ``dsa_workspace_bytes`` exists at once.
"""
from __future__ import annotations


import torch
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.models.draft.dflash import DFlashAttention
from aspec_b200.ops.attention import interval_attention
from aspec_b200.ops.linear import Linear
from aspec_b200.ops.norm import RMSNorm
from aspec_b200.ops.rope import qk_norm_rope


def _rotary(values: torch.Tensor, positions: torch.Tensor, dim: int, theta: float) -> torch.Tensor:
    """Non-interleaved RoPE on ``values[..., :dim]`` (``values [N, H, d]``)."""
    inv = theta ** (-torch.arange(0, dim, 2, device=values.device).float() / dim)
    ang = positions.float()[:, None] * inv
    cos, sin = ang.cos()[:, None], ang.sin()[:, None]
    a, b = values[..., :dim].float().chunk(2, -1)
    rot = torch.cat((a * cos - b * sin, a * sin + b * cos), -1).to(values.dtype)
    return torch.cat((rot, values[..., dim:]), -1)


def dist_all_gather(parts, tensor, group) -> None:
    import torch.distributed as dist
    dist.all_gather(parts, tensor, group=group)


def dist_all_reduce(tensor, group) -> None:
    import torch.distributed as dist
    dist.all_reduce(tensor, group=group)


class DSALightningIndexer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_heads, self.head_dim = config.dsa_index_n_heads, config.dsa_index_head_dim
        self.token_budget, self.workspace_bytes = config.dsa_token_budget, config.dsa_workspace_bytes
        self.rope_dim, self.rope_theta = config.dsa_rope_dim, config.dsa_rope_theta
        self.q_a_proj = Linear(config.hidden_size, config.dsa_q_lora_rank)
        self.q_a_norm = RMSNorm(config.dsa_q_lora_rank, eps=config.rms_norm_eps)
        self.q_b_proj = Linear(config.dsa_q_lora_rank, self.num_heads * self.head_dim)
        self.k_proj = Linear(config.hidden_size, self.head_dim)
        self.k_norm = nn.LayerNorm(self.head_dim, eps=config.rms_norm_eps)
        self.weights_proj = Linear(config.hidden_size, self.num_heads)
        self.scale = self.head_dim ** -0.5 * self.num_heads ** -0.5

    def project(self, x, ctx, q_pos, ctx_pos):
        x, ctx = x.detach(), ctx.detach()
        q = self.q_b_proj(self.q_a_norm(self.q_a_proj(x))).view(x.shape[0], self.num_heads, self.head_dim)
        kn = self.k_norm                     # statistics in fp32 whatever the module's parameter dtype
        k = F.layer_norm(self.k_proj(ctx).float(), kn.normalized_shape, kn.weight.float(), kn.bias.float(),
                         kn.eps).to(ctx.dtype)[:, None]
        q = _rotary(q, q_pos, self.rope_dim, self.rope_theta)
        k = _rotary(k, ctx_pos, self.rope_dim, self.rope_theta)[:, 0]
        w = F.linear(x.float(), self.weights_proj.weight.float()) * self.scale
        return q, k, w

    @staticmethod
    def scores(q, k, w):
        """``q [n, Hi, di]``, ``k [T, di]``, ``w [n, Hi]`` -> ``[n, T]`` fp32."""
        return (torch.einsum("nhd,td->nht", q.float(), k.float()).relu_() * w[:, :, None]).sum(1)

    def chunk_rows(self, n_keys: int) -> int:
        return max(int(self.workspace_bytes // max(n_keys * 4 * (self.num_heads + 2), 1)), 1)


class DSAAttention(DFlashAttention):
    def __init__(self, config, layer_idx: int):
        super().__init__(config, layer_idx)
        self.stage = config.dsa_training_stage
        self.indexer = DSALightningIndexer(config)
        self.compute_auxiliary_loss = True

    # teacher: head-summed softmax of the main attention over the eligible context --------------------
    def _teacher(self, q, k_ctx, lo, hi):
        g = self.num_heads // self.num_kv_heads
        kk = k_ctx.repeat_interleave(g, 1).float()
        s = torch.einsum("nhd,thd->nht", q.float(), kk) * self.scale
        t = torch.arange(k_ctx.shape[0], device=q.device)[None]
        elig = (t >= lo[:, None]) & (t < hi[:, None])
        s = s.masked_fill(~elig[:, None], float("-inf"))
        p = torch.softmax(s, -1)
        p = torch.where(elig[:, None], p, torch.zeros_like(p)).sum(1)
        return p / p.sum(-1, keepdim=True).clamp_min(1e-20), elig

    def forward(self, x, ctx, q_pos, kv_pos, intervals, aux=None, attn_override=None):
        if self.stage == "dense":
            return super().forward(x, ctx, q_pos, kv_pos, intervals, aux=aux, attn_override=attn_override)
        if isinstance(intervals, dict):
            if self.stage != "sparse":
                raise NotImplementedError("under context parallelism DSA runs its dense and sparse stages; warm the "
                                          "indexer up on one rank per row (draft_context_parallel_size=1)")
            return self._forward_context_parallel(x, ctx, q_pos, kv_pos, intervals, aux)
        Q, T = x.shape[0], ctx.shape[0]
        d, hk = self.head_dim, self.num_kv_heads
        from aspec_b200.ops.fused_params import fused_linear
        frozen = self.stage == "indexer_warmup"
        with torch.set_grad_enabled(torch.is_grad_enabled() and not frozen):
            q = self.q_proj(x).view(Q, self.num_heads, d)
            kv = fused_linear(torch.cat([ctx, x], 0), [self.k_proj.weight, self.v_proj.weight])
            k = kv[:, : hk * d].reshape(T + Q, hk, d)
            v = kv[:, hk * d:].reshape(T + Q, hk, d)
            inv = self.rope_freqs.get(x.device)
            q = qk_norm_rope(q, self.q_norm.weight, q_pos, inv, self.eps, self.rope_scaling)
            k = qk_norm_rope(k, self.k_norm.weight, kv_pos, inv, self.eps, self.rope_scaling)
        iq, ik, iw = self.indexer.project(x, ctx, q_pos, kv_pos[:T])
        lo, hi = intervals[:, 0].long(), intervals[:, 1].long()
        from aspec_b200.ops import sparse_attention as SA
        if self.stage == "sparse" and SA._kernel_ok(q, k, v):
            return self.o_proj(self._sparse_stage_kernels(q, k, v, iq, ik, iw, intervals, T, aux).reshape(Q, -1))
        rows = self.indexer.chunk_rows(T)
        losses = []
        outs = []
        budget = min(self.indexer.token_budget, T)
        for s0 in range(0, Q, rows):
            sl = slice(s0, min(s0 + rows, Q))
            score = self.indexer.scores(iq[sl], ik, iw[sl])
            with torch.no_grad():
                teacher, elig = self._teacher(q[sl].detach(), k[:T].detach(), lo[sl], hi[sl])
            if self.stage == "indexer_warmup":
                logp = torch.log_softmax(score.masked_fill(~elig, float("-inf")), -1)
                kl = (teacher * (torch.log(teacher.clamp_min(1e-20)) - logp.masked_fill(~elig, 0.0))).sum(-1)
                losses.append(torch.where(elig.any(-1), kl, torch.zeros_like(kl)))
                continue
            # sparse: per-query top-k over eligible context, KL on the selected set, attention on it + own block
            with torch.no_grad():
                masked = score.detach().masked_fill(~elig, float("-inf"))
                top = masked.topk(budget, -1)
                sel, sel_ok = top.indices, torch.isfinite(top.values)
            sel_score = score.gather(1, sel).masked_fill(~sel_ok, float("-inf"))
            t_sel = teacher.gather(1, sel) * sel_ok
            t_sel = t_sel / t_sel.sum(-1, keepdim=True).clamp_min(1e-20)
            logp = torch.log_softmax(sel_score, -1).masked_fill(~sel_ok, 0.0)
            kl = (t_sel * (torch.log(t_sel.clamp_min(1e-20)) - logp)).sum(-1)
            losses.append(torch.where(sel_ok.any(-1), kl, torch.zeros_like(kl)))
            outs.append(self._selected_attention(q[sl], k, v, sel, sel_ok, intervals[sl], T))
        if aux is not None and self.compute_auxiliary_loss and losses:
            aux.setdefault("dsa_losses", []).append(torch.cat(losses))
        if self.stage == "indexer_warmup":
            with torch.no_grad():
                o, _ = interval_attention(q, k, v, intervals, self.scale)
                return self.o_proj(o.reshape(Q, -1))
        return self.o_proj(torch.cat(outs, 0).reshape(Q, -1))

    def _sparse_stage_kernels(self, q, k, v, iq, ik, iw, intervals, T, aux):
        """The sparse stage on a GPU: indexer scores (tcgen05 GEMM with the ReLU / weight / head-sum epilogue), radix
        top-k and attention over the selected rows are kernels; nothing of size ``Q x T x heads`` is materialised.
        The KL between the main attention's and the indexer's distributions is taken on the selected set only, so
        its pieces - the selected indexer scores (with gradient) and the attention logits at the selected keys - are
        small gathers, chunked over queries; the per-head normaliser of the main attention over ALL eligible keys
        comes from one forward of the interval kernel."""
        from aspec_b200.ops import sparse_attention as SA
        from aspec_b200.models.draft.sparse_common import indexed_attention, own_block_index
        Q = q.shape[0]
        lo, hi = intervals[:, 0].contiguous(), intervals[:, 1].contiguous()
        budget = min(self.indexer.token_budget, T)
        rows = max(int(self.indexer.workspace_bytes // max(T * 4 * 2, 1)), 1)
        picks = []
        for s0 in range(0, Q, rows):
            sl = slice(s0, min(s0 + rows, Q))
            score = SA.indexer_scores(iq[sl].detach(), ik.detach(), iw[sl].detach(), lo[sl], hi[sl])
            picks.append(SA.topk_select(score, lo[sl], hi[sl], budget))
            del score
        sel = torch.cat(picks) if picks else torch.zeros(0, budget, dtype=torch.int32, device=q.device)
        if aux is not None and self.compute_auxiliary_loss:
            aux.setdefault("dsa_losses", []).append(self._selected_set_kl(q, k, iq, ik, iw, sel, intervals, T))
        blk, blk_ok = own_block_index(intervals, k.shape[0])
        idx = torch.cat([sel.long().clamp_min(0), blk], 1)
        ok = torch.cat([sel >= 0, blk_ok], 1)
        return indexed_attention(q, k, v, idx, ok, self.scale)

    @torch.no_grad()
    def _teacher_mass_on_selected(self, q, k_ctx, idx, ok, lse_rows):
        """Sum over heads of the main attention's probability of each selected key, ``[n, S]`` fp32.

        ``idx [n, S]`` indexes ``k_ctx [T, Hkv, d]`` (clamped; ``ok`` marks real entries); ``lse_rows [n, Hq]`` is the
        log-sum-exp of each query head over its whole eligible context (0 where empty).  Rows are processed in chunks
        sized by the indexer's workspace budget, and the key-head group is kept as a dimension instead of repeating the
        gathered keys per query head, so the transient is ``S x Hkv x d`` per row."""
        n, S = idx.shape
        hk, d = self.num_kv_heads, self.head_dim
        g = self.num_heads // hk
        per_row = S * (hk * d * 6 + self.num_heads * 8)
        rows = max(int(self.indexer.workspace_bytes // max(per_row, 1)), 1)
        out = torch.empty(n, S, dtype=torch.float32, device=q.device)
        for r0 in range(0, n, rows):
            sl = slice(r0, min(r0 + rows, n))
            kk = k_ctx[idx[sl]].float()                                               # [c, S, Hkv, d]
            qq = q[sl].float().reshape(-1, hk, g, d)
            logit = torch.einsum("nkgd,nskd->nkgs", qq, kk).reshape(qq.shape[0], hk * g, S) * self.scale
            out[sl] = (torch.exp(logit - lse_rows[sl][:, :, None]) * ok[sl][:, None]).sum(1)
        return out

    @staticmethod
    def _rows_of(table: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """``table[idx]`` in fp32 for an index tensor full of repeats, as ``index_select``: its backward is an
        ``index_add_`` (atomic adds), where advanced indexing's backward sorts the indices and walks every repeat of a
        row serially - measured 1.26 s per call against milliseconds for 7.3 M indices into 8 K rows on a B200."""
        flat = table.float().index_select(0, idx.reshape(-1))
        return flat.view(*idx.shape, *table.shape[1:])

    def _selected_set_kl(self, q, k, iq, ik, iw, sel, intervals, T):
        """``KL(teacher || indexer)`` per query over its selected keys.  teacher(s) is proportional to the sum over heads
        of the main attention's probability of key ``s`` under the softmax over the whole eligible context."""
        Q, S = sel.shape
        g = self.num_heads // self.num_kv_heads
        with torch.no_grad():
            ctx_only = torch.stack([intervals[:, 0], intervals[:, 1], torch.zeros_like(intervals[:, 0]),
                                    torch.zeros_like(intervals[:, 0])], 1).to(torch.int32).contiguous()
            _, lse = interval_attention(q.detach(), k[:T].detach(), k[:T].detach(), ctx_only, self.scale)   # [Hq, Q]
        per_row = S * (self.num_kv_heads * self.head_dim * 2 + self.num_heads * 4 * 2 + self.indexer.num_heads * 4 * 2)
        rows = max(int(self.indexer.workspace_bytes // max(per_row, 1)), 1)
        out = []
        for s0 in range(0, Q, rows):
            sl = slice(s0, min(s0 + rows, Q))
            s_idx = sel[sl].long().clamp_min(0)
            ok = sel[sl] >= 0
            sel_score = (torch.einsum("nhd,nsd->nhs", iq[sl].float(), self._rows_of(ik, s_idx)).relu() * iw[sl][:, :, None]).sum(1)
            with torch.no_grad():
                l = lse[:, sl].t()
                l = torch.where(torch.isfinite(l), l, torch.zeros_like(l))
                t_sel = self._teacher_mass_on_selected(q[sl].detach(), k[:T].detach(), s_idx, ok, l)
                t_sel = t_sel / t_sel.sum(-1, keepdim=True).clamp_min(1e-20)
            logp = torch.log_softmax(sel_score.masked_fill(~ok, float("-inf")), -1).masked_fill(~ok, 0.0)
            kl = (t_sel * (torch.log(t_sel.clamp_min(1e-20)) - logp)).sum(-1)
            out.append(torch.where(ok.any(-1), kl, torch.zeros_like(kl)))
        return torch.cat(out) if out else q.new_zeros(0, dtype=torch.float32)

    def _forward_context_parallel(self, x, ctx, q_pos, kv_pos, cpinfo, aux):
        """Sparse stage with the context sharded over the group (``ctx`` = this rank's shard, ``x`` = its own blocks).

        Queries and their indexer projections are gathered over the group; every rank scores all queries against ITS
        keys; the per-shard top-k candidates are merged into one global selection; each rank attends the selected keys
        it owns (the owner also its own block) and the partials are merged by log-sum-exp; the KL between the main
        attention and the indexer on the selected set is assembled from per-shard pieces with two small reductions.
        """
        from aspec_b200.ops import sparse_attention as SA
        from aspec_b200.ops.fused_params import fused_linear
        from aspec_b200.parallel.cp_runtime import _AllGatherStack, _pad_rows
        from aspec_b200.parallel.distributed_sparse import (_AllReduceSum, distributed_log_softmax,
                                                            distributed_selected_attention, distributed_topk,
                                                            split_selection)
        cp, counts, tables = cpinfo["cp"], list(cpinfo["counts"]), cpinfo["tables"]
        s0, s1, _total = cpinfo["shard"]
        group, rank = cp.group, cp.rank
        Q, T = x.shape[0], ctx.shape[0]
        d, hk = self.head_dim, self.num_kv_heads
        q = self.q_proj(x).view(Q, self.num_heads, d)
        kv = fused_linear(torch.cat([ctx, x], 0), [self.k_proj.weight, self.v_proj.weight])
        k = kv[:, : hk * d].reshape(T + Q, hk, d)
        v = kv[:, hk * d:].reshape(T + Q, hk, d)
        inv = self.rope_freqs.get(x.device)
        q = qk_norm_rope(q, self.q_norm.weight, q_pos, inv, self.eps, self.rope_scaling)
        k = qk_norm_rope(k, self.k_norm.weight, kv_pos, inv, self.eps, self.rope_scaling)
        iq, ik, iw = self.indexer.project(x, ctx, q_pos, kv_pos[:T])
        # -- gather the group's queries (padded to the largest owner), keep the valid rows in owner order ----------
        cap = max(max(counts), 1)
        valid = torch.cat([torch.arange(c, device=x.device) + o * cap for o, c in enumerate(counts)]) if sum(counts) else None
        def gather(t):
            rows = _AllGatherStack.apply(_pad_rows(t, cap), group).flatten(0, 1)
            return rows.index_select(0, valid) if valid is not None else rows[:0]
        q_all, iq_all, iw_all = gather(q), gather(iq), gather(iw)
        q_tot = q_all.shape[0]
        owner_lo = sum(counts[:rank])
        owner_hi = owner_lo + counts[rank]
        table_all = torch.cat([t for t in tables if t.shape[0]]) if q_tot else tables[rank]
        l_lo, l_hi = table_all[:, 0].contiguous(), table_all[:, 1].contiguous()        # eligible LOCAL key range
        # -- selection: local scores of all queries, global top-k ------------------------------------------------
        budget = self.indexer.token_budget
        with torch.no_grad():
            if T:
                score = SA.indexer_scores(iq_all.detach(), ik.detach(), iw_all.detach(), l_lo, l_hi)
            else:
                score = torch.zeros(q_tot, 0, device=x.device)
            sel = distributed_topk(score, l_lo.long() + s0, l_hi.long() + s0, budget, s0, group)      # global indices
            del score
        # -- attention over the selected keys of every shard + the query's own block on its owner ----------------
        own = tables[rank]
        width = int((own[:, 3] - own[:, 2]).max().item()) if own.shape[0] else 0
        extra = torch.full((q_tot, max(width, 1)), -1, dtype=torch.int32, device=x.device)
        if own.shape[0] and width:
            blk = own[:, 2:3].long() + torch.arange(width, device=x.device)[None]
            extra[owner_lo:owner_hi] = torch.where(blk < own[:, 3:4].long(), blk, torch.full_like(blk, -1)).to(torch.int32)
        out = distributed_selected_attention(q_all, k, v, sel, s0, owner_lo, owner_hi, self.scale, group, extra_local=extra,
                                             shard_len=T)
        # -- KL(main attention || indexer) on the selected set, assembled over shards -----------------------------
        if aux is not None and self.compute_auxiliary_loss:
            local = split_selection(sel, s0, s0 + T).long()
            ok = local >= 0
            safe = local.clamp_min(0)
            if T:
                sel_score = (torch.einsum("nhd,nsd->nhs", iq_all.float(), self._rows_of(ik, safe)).relu() * iw_all[:, :, None]).sum(1)
            else:
                sel_score = torch.zeros(q_tot, local.shape[1], device=x.device) + 0.0 * iq_all.float().sum()
            logp, _ = distributed_log_softmax(sel_score, ok, group)
            with torch.no_grad():
                g = self.num_heads // self.num_kv_heads
                ctx_only = torch.stack([l_lo, l_hi, torch.zeros_like(l_lo), torch.zeros_like(l_lo)], 1).to(torch.int32).contiguous()
                if T:
                    _, lse_loc = interval_attention(q_all.detach(), k[:T].detach(), k[:T].detach(), ctx_only, self.scale)
                    lse_loc = lse_loc.float()
                else:
                    lse_loc = torch.full((self.num_heads, q_tot), float("-inf"), device=x.device)
                parts = [torch.empty_like(lse_loc) for _ in range(cp.size)]
                dist_all_gather(parts, lse_loc.contiguous(), group)
                lse = torch.logsumexp(torch.stack(parts), 0)                                 # [Hq, Q_tot] over all shards
                lse = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse)).t()
                if T:
                    t_loc = self._teacher_mass_on_selected(q_all.detach(), k[:T].detach(), safe, ok, lse)
                else:
                    t_loc = torch.zeros(q_tot, local.shape[1], device=x.device)
                z = t_loc.sum(-1)
                dist_all_reduce(z, group)
                t_sel = t_loc / z.clamp_min(1e-20)[:, None]
            kl_part = (t_sel * (torch.log(t_sel.clamp_min(1e-20)) - logp) * ok).sum(-1)
            kl = _AllReduceSum.apply(kl_part, group)
            aux.setdefault("dsa_losses", []).append(torch.where(z > 0, kl, torch.zeros_like(kl))[owner_lo:owner_hi])
        return self.o_proj(out.reshape(Q, -1))

    def _selected_attention(self, q, k, v, sel, sel_ok, iv, T):
        """Each query attends its selected context tokens and the whole of its own draft block."""
        n = q.shape[0]
        g = self.num_heads // self.num_kv_heads
        b_lo, b_hi = iv[:, 2].long(), iv[:, 3].long()
        width = int((b_hi - b_lo).max().item()) if n else 0
        off = torch.arange(width, device=q.device)[None]
        blk = b_lo[:, None] + off
        blk_ok = blk < b_hi[:, None]
        idx = torch.cat([sel, blk.clamp(max=k.shape[0] - 1)], 1)
        ok = torch.cat([sel_ok, blk_ok], 1)
        kk = k[idx].repeat_interleave(g, 2).float()              # [n, S, Hq, d]
        vv = v[idx].repeat_interleave(g, 2).float()
        s = torch.einsum("nhd,nshd->nhs", q.float(), kk) * self.scale
        s = s.masked_fill(~ok[:, None], float("-inf"))
        p = torch.softmax(s, -1)
        p = torch.where(ok[:, None], p, torch.zeros_like(p))
        return torch.einsum("nhs,nshd->nhd", p, vv).to(q.dtype)

    def trainable_parameter_names(self):
        """In ``indexer_warmup`` only the indexer learns (weights-only phase changes between stages)."""
        return [n for n, _ in self.named_parameters() if n.startswith("indexer.")] if self.stage == "indexer_warmup" else None
