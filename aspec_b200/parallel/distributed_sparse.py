"""Sparse attention when the context is sharded over a context-parallel group.

Every rank owns a contiguous shard ``[shard_lo, shard_hi)`` of the key rows and a subset of the queries.  The three
pieces the sparse drafts need (reference: aspec/models/ops/distributed_sparse.py:54-241,
aspec/models/ops/compact_varlen.py:205-256), restated for this framework:

* :func:`distributed_topk` - global top-k per query from per-shard scores.  A rank's local top-k is a superset of its
  share of the global top-k, so each rank sends only ``k`` candidates (value, global index) per query; the candidates
  are all-gathered and every rank takes the same global top-k (ties: lower global index first, so all ranks agree).
* :func:`distributed_log_softmax` - log-softmax over entries that live on different ranks: MAX then SUM all-reduce of the
  per-row statistics; differentiable (the gradient of the normaliser flows back through the SUM).
* :func:`distributed_selected_attention` - each rank attends, for ALL queries of the group, the selected keys it owns
  (the selected-key kernel on a GPU), and the partial outputs are merged exactly with their log-sum-exps at the query's
  owner.  Ranks whose shard holds none of a query's keys contribute ``lse = -inf``; ranks with an empty shard still
  join every collective.

Collectives here are ``torch.distributed`` calls (gloo on CPU, NCCL on GPUs): the messages are statistics and index
lists, not the bulk key / value traffic, which never leaves its owner.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from aspec_b200.ops.attention import merge_partials
from aspec_b200.ops.sparse_attention import topk_select


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


class _AllGatherCat(torch.autograd.Function):
    """Concatenate every rank's ``[n, m]`` block along the last dim; backward returns this rank's slice of the summed gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.m = group, x.shape[-1]
        parts = [torch.empty_like(x) for _ in range(_world(group))]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, -1)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        return g[..., r * ctx.m:(r + 1) * ctx.m], None


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


@torch.no_grad()
def distributed_topk(local_scores: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, k: int, shard_lo: int,
                     group=None) -> torch.Tensor:
    """Global indices ``[n, k]`` (ascending, ``-1`` padded) of the ``k`` best keys of every query over all shards.

    ``local_scores [n, T_loc]`` are this rank's scores of all ``n`` queries against its own keys; ``lo / hi [n]`` the
    eligible GLOBAL key range of each query; ``shard_lo`` the global index of this rank's first key.
    """
    n, t_loc = local_scores.shape
    dev = local_scores.device
    l_lo = (lo.long() - shard_lo).clamp(0, t_loc)
    l_hi = (hi.long() - shard_lo).clamp(0, t_loc)
    if t_loc:
        loc = topk_select(local_scores.float().contiguous(), l_lo, l_hi, k).long()            # local indices, -1 padded
    else:
        loc = torch.full((n, k), -1, dtype=torch.long, device=dev)
    ok = loc >= 0
    vals = torch.where(ok, local_scores.float().gather(1, loc.clamp_min(0)) if t_loc else loc.float(),
                       torch.full((n, k), float("-inf"), device=dev))
    gidx = torch.where(ok, loc + shard_lo, torch.full_like(loc, -1))
    if _world(group) > 1:
        all_v = [torch.empty_like(vals) for _ in range(_world(group))]
        all_i = [torch.empty_like(gidx) for _ in range(_world(group))]
        dist.all_gather(all_v, vals.contiguous(), group=group)
        dist.all_gather(all_i, gidx.contiguous(), group=group)
        vals, gidx = torch.cat(all_v, 1), torch.cat(all_i, 1)
    # global selection among the candidates; ties broken by the lower global index so that every rank agrees
    big = torch.iinfo(torch.long).max
    order = torch.argsort(torch.where(gidx >= 0, gidx, torch.full_like(gidx, big)), dim=1, stable=True)
    vals, gidx = vals.gather(1, order), gidx.gather(1, order)
    pick = torch.argsort(vals, dim=1, descending=True, stable=True)[:, :k]
    chosen_v, chosen_i = vals.gather(1, pick), gidx.gather(1, pick)
    chosen_i = torch.where(torch.isfinite(chosen_v), chosen_i, torch.full_like(chosen_i, -1))
    # ascending index order, empty slots last
    key = torch.where(chosen_i >= 0, chosen_i, torch.full_like(chosen_i, big))
    return chosen_i.gather(1, torch.argsort(key, dim=1, stable=True)).to(torch.int32)


def distributed_log_softmax(local_logits: torch.Tensor, mask: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Log-softmax over the union of every rank's masked entries of each row.

    ``local_logits [n, S_loc]`` with validity ``mask``; returns ``(log_prob [n, S_loc]`` (0 where masked), ``valid [n]``
    true when any rank has an entry for the row).  Differentiable in ``local_logits``.
    """
    x = local_logits.float().masked_fill(~mask, float("-inf"))
    row_max = x.max(-1).values if x.shape[-1] else x.new_full((x.shape[0],), float("-inf"))
    with torch.no_grad():
        m = row_max.detach().clone()
        if _world(group) > 1:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        valid = torch.isfinite(m)
        m = torch.where(valid, m, torch.zeros_like(m))
    e = torch.where(mask, torch.exp(x - m[:, None]), torch.zeros_like(x))
    total = e.sum(-1)
    if _world(group) > 1:
        total = _AllReduceSum.apply(total, group)
    log_z = torch.log(total.clamp_min(1e-30)) + m
    logp = torch.where(mask, x - log_z[:, None], torch.zeros_like(x))
    return logp, valid


def split_selection(sel_global: torch.Tensor, shard_lo: int, shard_hi: int) -> torch.Tensor:
    """The entries of a global selection that this shard owns, as local indices (``-1`` elsewhere)."""
    s = sel_global.long()
    mine = (s >= shard_lo) & (s < shard_hi)
    return torch.where(mine, s - shard_lo, torch.full_like(s, -1)).to(torch.int32)


class _ShardedSelectedAttention(torch.autograd.Function):
    """Forward: this shard's partial, all-gather of partials, exact merge (every rank ends up with every query's merged
    output and global log-sum-exp).  Backward: the owners' output gradients are gathered and each rank runs the ordinary
    selected-key backward on ITS keys with the GLOBAL output and log-sum-exp - probabilities are then those of the whole
    softmax and the three gradients are this shard's exact share; nothing has to be differentiated through the merge."""

    @staticmethod
    def forward(ctx, q_all, k_local, v_local, local_sel, scale, group, owner_lo, owner_hi):
        from aspec_b200.ops.sparse_attention import selected_attention_forward
        n, hq, d = q_all.shape
        if k_local.shape[0]:
            part_o, part_l = selected_attention_forward(q_all, k_local, v_local, local_sel, scale)
        else:                   # an empty shard still joins every collective
            part_o = q_all.new_zeros(q_all.shape)
            part_l = q_all.new_full((hq, n), float("-inf"), dtype=torch.float32)
        part_l = part_l.float()
        if _world(group) > 1:
            all_o = [torch.empty_like(part_o) for _ in range(_world(group))]
            all_l = [torch.empty_like(part_l) for _ in range(_world(group))]
            dist.all_gather(all_o, part_o.contiguous(), group=group)
            dist.all_gather(all_l, part_l.contiguous(), group=group)
            out_all, lse_all = merge_partials(torch.stack(all_o), torch.stack(all_l))
        else:
            out_all, lse_all = part_o, part_l
        ctx.save_for_backward(q_all, k_local, v_local, local_sel, out_all, lse_all)
        ctx.scale, ctx.group, ctx.rows = scale, group, (owner_lo, owner_hi)
        return out_all[owner_lo:owner_hi].clone()

    @staticmethod
    def backward(ctx, dout_rows):
        from aspec_b200.ops.sparse_attention import selected_attention_backward
        q_all, k_local, v_local, local_sel, out_all, lse_all = ctx.saved_tensors
        lo, hi = ctx.rows
        dout_all = torch.zeros_like(out_all)
        dout_all[lo:hi] = dout_rows
        if _world(ctx.group) > 1:
            dist.all_reduce(dout_all, group=ctx.group)           # owners' rows are disjoint: the sum is the gather
        if k_local.shape[0]:
            dq, dk, dv = selected_attention_backward(q_all, k_local, v_local, local_sel, out_all, lse_all, dout_all, ctx.scale)
        else:
            dq, dk, dv = torch.zeros_like(q_all), torch.zeros_like(k_local, dtype=torch.float32), torch.zeros_like(v_local, dtype=torch.float32)
        # dq is this shard's share for EVERY query: whoever gathered the queries sums the shares in its own backward
        return dq.to(q_all.dtype), dk.to(k_local.dtype), dv.to(v_local.dtype), None, None, None, None, None


def distributed_selected_attention(q_all: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                                   sel_global: torch.Tensor, shard_lo: int, owner_lo: int, owner_hi: int, scale: float,
                                   group=None, extra_local: Optional[torch.Tensor] = None,
                                   shard_len: Optional[int] = None) -> torch.Tensor:
    """Attention of the group's queries over globally selected keys that are spread over the shards.

    ``q_all [Q_tot, H, d]``: all queries of the group (gathered by the caller, whose gather sums the per-rank query
    gradients in its backward); ``k_local / v_local [T_loc, Hk, d]``: this rank's keys; ``sel_global [Q_tot, S]`` global
    key indices (``-1`` = none); ``[owner_lo, owner_hi)``: the rows of ``q_all`` this rank owns and whose merged outputs
    it returns.  ``extra_local [Q_tot, E]``: more LOCAL indices every query attends on this rank (for example its own
    draft block on the owner; ``-1`` elsewhere).  ``shard_len``: how many leading rows of ``k_local`` are the context
    shard that ``sel_global`` indexes (default: all of them; the rest are rows only ``extra_local`` can name).
    Returns ``out [owner_hi - owner_lo, H, d]``.
    """
    t_loc = k_local.shape[0] if shard_len is None else int(shard_len)
    local = split_selection(sel_global, shard_lo, shard_lo + t_loc)
    if extra_local is not None:
        local = torch.cat([local, extra_local.to(torch.int32)], 1)
    return _ShardedSelectedAttention.apply(q_all, k_local, v_local, local.contiguous(), float(scale), group,
                                           int(owner_lo), int(owner_hi))
