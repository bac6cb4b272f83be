"""Ring attention over a sequence that is sharded contiguously among the ranks of a group.

Rank ``r`` owns key / value rows ``[r S, (r + 1) S)`` of the ring-distributed sequence (plus, optionally, extra rows
that only its own queries may attend: a Draft block, or the test-time-training keys of EAGLE).  Its queries attend keys
anywhere in the sequence.  K / V blocks travel once around the ring; at every stop the resident queries attend the
visiting block with the interval kernel, and the partial results are merged exactly through their log-sum-exps.

The backward pass walks the ring again: each stop runs the ordinary attention backward on the visiting block with the
GLOBAL output and log-sum-exp of the queries (the probabilities are then those of the whole softmax, so every stop's
``dQ``, ``dK``, ``dV`` are exact shares); ``dK`` / ``dV`` travel with their block and one last hop brings them home.

This is the ring stage of Ulysses x ring sequence parallelism (reference: aspec/models/draft/llama3_eagle.py:1925-2034,
which drives yunchang's ring flash-attention and merges the extra-key terms with ``logaddexp``).  Block transfers are
``torch.distributed`` point-to-point operations (NCCL on GPUs, gloo on CPU), posted before the stop's attention is
launched so that the transfer overlaps the compute of the current block.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from aspec_b200.ops.attention import interval_attention_reference


def _size(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def shard_intervals(intervals: torch.Tensor, owner: int, shard_rows: int, keep_local: bool) -> torch.Tensor:
    """Global table ``[a0, a1, b0, b1]`` -> the table against the key array ``[owner's shard | local extra rows]``.

    ``[a0, a1)`` is in ring coordinates ``[0, R S)`` and is clipped to the owner's shard; ``[b0, b1)`` indexes the extra
    rows (already relative to the local key array) and is kept only on the queries' own rank."""
    iv = intervals.to(torch.int64)
    lo = owner * shard_rows
    a0 = iv[:, 0].clamp(lo, lo + shard_rows) - lo
    a1 = torch.maximum(iv[:, 1].clamp(lo, lo + shard_rows) - lo, a0)
    if keep_local:
        b0, b1 = iv[:, 2], iv[:, 3]
    else:
        b0 = b1 = torch.zeros_like(a0)
    return torch.stack([a0, a1, b0, b1], -1).to(torch.int32).contiguous()


def _forward_partial(q, k, v, iv, scale) -> Tuple[torch.Tensor, torch.Tensor]:
    if q.is_cuda:
        from aspec_b200.ops import attention_sm100 as K
        if K.supported(q, k, v):
            return K.forward(q, k, v, iv, scale)
    out, lse = interval_attention_reference(q, k, v, iv, scale)
    return out, lse.float()


def interval_attention_backward_reference(q, k, v, iv, out, lse, dout, scale):
    """fp32 backward of interval attention given ``out`` / ``lse [Hq, Q]`` (possibly those of a larger softmax)."""
    from aspec_b200.ops.attention import dense_interval_mask
    g = q.shape[1] // k.shape[1]
    qf, do = q.float().transpose(0, 1), dout.float().transpose(0, 1)              # [Hq, Q, d]
    kf = k.float().transpose(0, 1).repeat_interleave(g, 0)                        # [Hq, Tk, d]
    vf = v.float().transpose(0, 1).repeat_interleave(g, 0)
    vis = dense_interval_mask(iv, k.shape[0])[None]
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    l = lse.float()
    has = torch.isfinite(l)
    p = torch.exp(s - torch.where(has, l, torch.zeros_like(l))[..., None])
    p = torch.where(vis & has[..., None], p, torch.zeros_like(p))
    delta = (out.float().transpose(0, 1) * do).sum(-1)                            # [Hq, Q]
    dp = torch.matmul(do, vf.transpose(1, 2))
    ds = p * (dp - delta[..., None]) * scale
    dq = torch.matmul(ds, kf).transpose(0, 1)
    dk = torch.matmul(ds.transpose(1, 2), qf).reshape(k.shape[1], g, k.shape[0], -1).sum(1).transpose(0, 1)
    dv = torch.matmul(p.transpose(1, 2), do).reshape(k.shape[1], g, k.shape[0], -1).sum(1).transpose(0, 1)
    return dq, dk, dv


def _backward_partial(q, k, v, iv, out, lse, dout, scale):
    if q.is_cuda:
        from aspec_b200.ops import attention_sm100 as K
        if K.supported(q, k, v):
            dq, dk, dv = K.backward(q, k, v, iv, out, lse.float().contiguous(), dout, scale)
            return dq.float(), dk.float(), dv.float()
    return interval_attention_backward_reference(q, k, v, iv, out, lse, dout, scale)


def _merge(out, lse, part_o, part_l):
    """Exact pairwise merge of two partial attentions over disjoint key sets (``lse [Hq, Q]``, ``out [Q, Hq, d]``)."""
    if out is None:
        return part_o.float(), part_l.float()
    new = torch.logaddexp(lse, part_l.float())
    safe = torch.where(torch.isfinite(new), new, torch.zeros_like(new))
    w_old = torch.where(torch.isfinite(lse), torch.exp(lse - safe), torch.zeros_like(lse))
    w_new = torch.where(torch.isfinite(part_l), torch.exp(part_l.float() - safe), torch.zeros_like(new))
    merged = out * w_old.t()[..., None] + part_o.float() * w_new.t()[..., None]
    return merged, new


class _Hop:
    """One hop of the ring: every tensor of ``blocks`` goes to the next rank while the previous rank's arrive."""

    def __init__(self, blocks, group):
        self.blocks, self.recv, self.reqs = blocks, None, None
        size, rank = _size(group), _rank(group)
        if size == 1:
            self.recv = blocks
            return
        nxt = dist.get_global_rank(group, (rank + 1) % size) if group is not None else (rank + 1) % size
        prv = dist.get_global_rank(group, (rank - 1) % size) if group is not None else (rank - 1) % size
        self.recv = [torch.empty_like(b) for b in blocks]
        ops = []
        for b, r in zip(blocks, self.recv):
            ops.append(dist.P2POp(dist.isend, b.contiguous(), nxt, group))
            ops.append(dist.P2POp(dist.irecv, r, prv, group))
        self.reqs = dist.batch_isend_irecv(ops)

    def wait(self):
        if self.reqs is not None:
            for r in self.reqs:
                r.wait()
        return self.recv


class _RingAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k_local, v_local, intervals, shard_rows, scale, group):
        R, r = _size(group), _rank(group)
        S = int(shard_rows)
        out = lse = None
        k_cur, v_cur = k_local[:S].contiguous(), v_local[:S].contiguous()
        for step in range(R):
            owner = (r - step) % R
            hop = _Hop([k_cur, v_cur], group) if step < R - 1 else None       # posted first: overlaps this stop's attention
            iv = shard_intervals(intervals, owner, S, keep_local=(step == 0))
            keys, vals = (k_local, v_local) if step == 0 else (k_cur, v_cur)
            part_o, part_l = _forward_partial(q, keys, vals, iv, scale)
            out, lse = _merge(out, lse, part_o, part_l)
            if hop is not None:
                k_cur, v_cur = hop.wait()
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k_local, v_local, intervals, out, lse)
        ctx.meta = (S, scale, group)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k_local, v_local, intervals, out, lse = ctx.saved_tensors
        S, scale, group = ctx.meta
        R, r = _size(group), _rank(group)
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dk_local = torch.zeros(k_local.shape, dtype=torch.float32, device=q.device)
        dv_local = torch.zeros(v_local.shape, dtype=torch.float32, device=q.device)
        k_cur, v_cur = k_local[:S].contiguous(), v_local[:S].contiguous()
        dk_cur = dv_cur = None
        for step in range(R):
            owner = (r - step) % R
            hop = _Hop([k_cur, v_cur], group) if step < R - 1 else None
            iv = shard_intervals(intervals, owner, S, keep_local=(step == 0))
            if step == 0:
                dq_p, dk_p, dv_p = _backward_partial(q, k_local, v_local, iv, out, lse, dout, scale)
                dk_local[S:] += dk_p[S:]
                dv_local[S:] += dv_p[S:]
                dk_cur, dv_cur = dk_p[:S].contiguous(), dv_p[:S].contiguous()
            else:
                dq_p, dk_p, dv_p = _backward_partial(q, k_cur, v_cur, iv, out, lse, dout, scale)
                dk_cur, dv_cur = dk_cur + dk_p, dv_cur + dv_p
            dq += dq_p
            if hop is not None:
                k_cur, v_cur = hop.wait()
                dk_cur, dv_cur = _Hop([dk_cur, dv_cur], group).wait()        # gradients travel with their block
        if R > 1:
            dk_cur, dv_cur = _Hop([dk_cur, dv_cur], group).wait()            # the last hop brings them home
        dk_local[:S] += dk_cur
        dv_local[:S] += dv_cur
        return dq.to(q.dtype), dk_local.to(k_local.dtype), dv_local.to(v_local.dtype), None, None, None, None


def ring_attention(q: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor, intervals: torch.Tensor,
                   shard_rows: int, scale: float, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(out [Q, Hq, d], lse [Hq, Q])`` of this rank's queries over the whole ring-distributed sequence.

    ``k_local / v_local [S + E, Hk, d]``: this rank's ``S = shard_rows`` rows of the sequence, then ``E`` local-only rows;
    ``intervals [Q, 4]``: ``[a0, a1)`` in ring coordinates ``[0, R S)``, ``[b0, b1)`` in local key coordinates (``>= S``).
    Every rank of ``group`` must call this with the same ``shard_rows`` (pad the last shard)."""
    return _RingAttentionFn.apply(q, k_local, v_local, intervals.contiguous(), int(shard_rows), float(scale), group)
