"""Vocabulary-parallel output head with the softmax statistics merged over peer memory.

The frozen Target head ``W [V, D]`` (and the Markov projection ``[V, r]``) is split by rows over the ``p`` ranks of
a vocabulary-parallel group; every rank of the group holds the same supervised rows.  The reference replicates the
head on every trainer (aspec/training/dflash_trainer.py:303-310, aspec/models/dspark.py:553-636); this is new
capability.  Per call and rank:

1. ``logits_r = hidden @ W_r^T (+ prev_emb @ M_r^T)`` and the teacher's ``t_r`` on the tcgen05 GEMM whose epilogue
   emits per-tile (max, sum-exp); the rank's partial log-sum-exp vectors go to its peer-visible workspace;
2. every rank reads all ``p`` partial vectors straight from the peers' HBM and forms the global normalisers, runs the
   statistics pass of the loss kernel on its columns (partial CE term, ``sum|p-q|``, ``sum p*sign(p-q)``, arg-max)
   and publishes them the same way;
3. the partials are summed over the peers, the gradient pass overwrites ``logits_r`` with ``d loss / d logits_r``;
4. backward: ``dhidden_r = dlogits_r @ W_r`` is written by the GEMM epilogue into slot ``r`` of EVERY rank's slot
   buffer (peer stores, tile by tile while the GEMM runs); after the barrier each rank sums its ``p`` local slots.

No ``[R, V]`` tensor ever crosses NVLink: only ``O(R)`` statistics and the ``[R, D]`` partial gradients do.
The phases are separate methods so that several ranks can be emulated in one process (tests); ``barrier`` is a
tiny stream-ordered collective in real runs.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from aspec_b200.parallel.symmetric_memory import SymmetricBuffer


def _up(n: int, a: int = 256) -> int:
    return -(-n // a) * a


class VocabShardWorkspace:
    """Peer-visible scratch of one rank.  ``fields`` are views of one symmetric allocation."""

    def __init__(self, max_rows: int, max_teacher_rows: int, hidden: int, markov_rank: int, world: int, device=None,
                 buffer: Optional[SymmetricBuffer] = None):
        self.max_rows, self.max_teacher_rows, self.hidden, self.markov_rank, self.world = max_rows, max_teacher_rows, hidden, markov_rank, world
        sizes = [("lse_s", max_rows * 4), ("lse_t", max_teacher_rows * 4), ("stats", 3 * max_rows * 4),
                 ("best_val", max_rows * 4), ("best_idx", max_rows * 4), ("dh", world * max_rows * hidden * 2),
                 ("dprev", world * max_rows * max(markov_rank, 8) * 2)]
        self._offsets, off = {}, 0
        for name, n in sizes:
            self._offsets[name] = (off, n)
            off += _up(n)
        self.nbytes = off
        self.buffer = buffer if buffer is not None else SymmetricBuffer.allocate(off, device)
        raw = self.buffer.tensor
        v = lambda name, dt: raw[self._offsets[name][0]: self._offsets[name][0] + self._offsets[name][1]].view(dt)
        self.lse_s, self.lse_t = v("lse_s", torch.float32), v("lse_t", torch.float32)
        self.stats = v("stats", torch.float32).view(3, max_rows)
        self.best_val, self.best_idx = v("best_val", torch.float32), v("best_idx", torch.int32)
        self.dh = v("dh", torch.bfloat16).view(world, max_rows, hidden)
        self.dprev = v("dprev", torch.bfloat16).view(world, max_rows, max(markov_rank, 8))

    def export(self) -> dict:
        return {"memory": self.buffer.export(), "max_rows": self.max_rows, "max_teacher_rows": self.max_teacher_rows,
                "hidden": self.hidden, "markov_rank": self.markov_rank, "world": self.world}

    @classmethod
    def open(cls, meta: dict) -> "VocabShardWorkspace":
        return cls(meta["max_rows"], meta["max_teacher_rows"], meta["hidden"], meta["markov_rank"], meta["world"],
                   buffer=SymmetricBuffer.open(meta["memory"]))


class VocabParallelHead:
    def __init__(self, rank: int, world: int, vocab_size: int, workspaces: Sequence[VocabShardWorkspace],
                 barrier: Optional[Callable[[], None]] = None):
        if vocab_size % world or (vocab_size // world) % 8:
            raise ValueError("vocab_size must split into shards that are multiples of 8")
        self.rank, self.world, self.vocab = rank, world, vocab_size
        self.shard = vocab_size // world
        self.offset = rank * self.shard
        self.ws = list(workspaces)                 # index = rank; ws[rank] is this rank's own
        self.mine = self.ws[rank]
        self.barrier = barrier or (lambda: None)

    def shard_rows(self, weight: torch.Tensor) -> torch.Tensor:
        return weight[self.offset: self.offset + self.shard]

    # -- forward phases -----------------------------------------------------------------------------------
    def logits(self, hidden, w_shard, prev_emb=None, w2_shard=None, teacher_hidden=None, teacher_w_shard=None):
        from aspec_b200.ops import elementwise_sm100 as E
        from aspec_b200.ops import gemm as G
        R, dev = hidden.shape[0], hidden.device
        nt = -(-self.shard // G.TILE_N)
        stats = torch.empty(nt, R, 2, dtype=torch.float32, device=dev)
        self._logits = torch.empty(R, self.shard, dtype=torch.bfloat16, device=dev)
        G.gemm(hidden, w_shard, a2=prev_emb, b2=w2_shard, out=self._logits, epilogue=G.EPI_ROWSTATS, stats=stats)
        self.mine.lse_s[:R].copy_(E.merge_rowstats(stats))
        self._t_logits = None
        if teacher_hidden is not None:
            Tt = teacher_hidden.shape[0]
            t_stats = torch.empty(nt, Tt, 2, dtype=torch.float32, device=dev)
            self._t_logits = torch.empty(Tt, self.shard, dtype=torch.bfloat16, device=dev)
            G.gemm(teacher_hidden, w_shard if teacher_w_shard is None else teacher_w_shard, out=self._t_logits,
                   epilogue=G.EPI_ROWSTATS, stats=t_stats)
            self.mine.lse_t[:Tt].copy_(E.merge_rowstats(t_stats))
        self._R, self._Tt = R, (teacher_hidden.shape[0] if teacher_hidden is not None else 0)

    def statistics(self, labels, weight, t_index, a_ce: float, a_l1: float):
        from aspec_b200.ops import comm
        from aspec_b200.ops import elementwise_sm100 as E
        R, Tt, dev = self._R, self._Tt, self._logits.device
        self._lse_s = comm.peer_lse_merge([w.lse_s[:R] for w in self.ws], torch.empty(R, dtype=torch.float32, device=dev))
        self._lse_t = (comm.peer_lse_merge([w.lse_t[:Tt] for w in self.ws], torch.empty(Tt, dtype=torch.float32, device=dev))
                       if Tt else None)
        self._args = (labels, weight, t_index, a_ce, a_l1)
        m = self.mine
        E.vocab_loss_shard(self._logits, self._t_logits, self._lse_s, self._lse_t, t_index, labels, weight,
                           m.stats[0, :R], m.stats[1, :R], m.stats[2, :R], m.best_val[:R], m.best_idx[:R],
                           vocab_offset=self.offset, a_ce=a_ce, a_l1=a_l1 if Tt else 0.0, phase=1)

    def gradient(self, need_grad: bool = True):
        """Returns ``(ce, l1, correct)`` per row; ``self.dlogits`` then holds this shard's logit gradient."""
        from aspec_b200.ops import comm
        from aspec_b200.ops import elementwise_sm100 as E
        R, dev = self._R, self._logits.device
        labels, weight, t_index, a_ce, a_l1 = self._args
        rows4 = -(-R // 4) * 4
        total = torch.empty(3, rows4, dtype=torch.float32, device=dev)
        for k in range(3):
            comm.peer_reduce([w.stats[k, :rows4] for w in self.ws], total[k])
        ce = self._lse_s + total[0, :R]
        l1 = total[1, :R].clone()
        correct = comm.peer_argmax_merge([w.best_val[:R] for w in self.ws], [w.best_idx[:R] for w in self.ws], labels,
                                         torch.empty(R, dtype=torch.float32, device=dev))
        if need_grad:
            c = total[2, :R].contiguous()
            E.vocab_loss_shard(self._logits, self._t_logits, self._lse_s, self._lse_t, t_index, labels, weight,
                               self.mine.stats[0, :R], self.mine.stats[1, :R], c, self.mine.best_val[:R], self.mine.best_idx[:R],
                               vocab_offset=self.offset, a_ce=a_ce, a_l1=a_l1 if self._Tt else 0.0, phase=2)
        self.dlogits = self._logits
        self._t_logits = None
        return ce, l1, correct

    # -- backward phases ----------------------------------------------------------------------------------
    def scatter_partials(self, w_shard, w2_shard=None):
        """``dlogits_r @ W_r`` (and ``@ M_r``) stored by the GEMM epilogue into slot ``rank`` of every rank's buffer."""
        from aspec_b200.ops import gemm as G
        R = self._R
        slots = [w.dh[self.rank, :R] for w in self.ws]
        G.gemm(self.dlogits, w_shard, b_t=True, out=slots[self.rank], mirrors=[s for i, s in enumerate(slots) if i != self.rank])
        if w2_shard is not None:
            rk = w2_shard.shape[1]
            slots = [w.dprev[self.rank, :R, :rk] for w in self.ws]
            G.gemm(self.dlogits, w2_shard, b_t=True, out=slots[self.rank], mirrors=[s for i, s in enumerate(slots) if i != self.rank])

    def reduce_partials(self, markov_rank: int = 0):
        from aspec_b200.ops import comm
        R, m = self._R, self.mine
        D = m.hidden
        dh = torch.empty(R, D, dtype=torch.bfloat16, device=m.dh.device)
        comm.peer_reduce([m.dh[r, :R].reshape(-1) for r in range(self.world)], dh.view(-1))
        dprev = None
        if markov_rank:
            full = torch.empty(R, m.dprev.shape[-1], dtype=torch.bfloat16, device=dh.device)
            comm.peer_reduce([m.dprev[r, :R].reshape(-1) for r in range(self.world)], full.view(-1))
            dprev = full[:, :markov_rank].contiguous()
        return dh, dprev


class _VocabParallelLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, head: VocabParallelHead, hidden, w_shard, prev_emb, w2_shard, teacher_hidden, t_index, labels,
                weight, a_ce, a_l1, w2_holder):
        head.logits(hidden, w_shard, prev_emb, w2_shard, teacher_hidden)
        head.barrier()
        head.statistics(labels, weight, t_index, a_ce, a_l1)
        head.barrier()
        ce, l1, correct = head.gradient(need_grad=True)
        num = (weight * (a_ce * ce + a_l1 * l1)).sum()
        ctx.head, ctx.w2_holder = head, w2_holder
        ctx.save_for_backward(hidden, w_shard, prev_emb, w2_shard)
        ctx.mark_non_differentiable(ce, l1, correct)
        return num, ce, l1, correct

    @staticmethod
    def backward(ctx, dnum, *_unused):
        from aspec_b200.ops import elementwise_sm100 as E
        from aspec_b200.ops import gemm as G
        head = ctx.head
        hidden, w_shard, prev_emb, w2_shard = ctx.saved_tensors
        scale = dnum.float().reshape(1)
        head.scatter_partials(w_shard, w2_shard if prev_emb is not None else None)
        head.barrier()
        dh, dprev = head.reduce_partials(prev_emb.shape[1] if prev_emb is not None else 0)
        E.scale_bf16_(dh, scale)
        if dprev is not None:
            E.scale_bf16_(dprev, scale)
        dw2 = None
        if prev_emb is not None and ctx.needs_input_grad[4]:
            g = G.gemm(head.dlogits, prev_emb, a_t=True, b_t=True, out_dtype=torch.float32)
            # every rank of the group back-propagates the same rows, and the data-parallel reduction then sums the
            # group's (otherwise identical) gradients: shard-only gradients are pre-multiplied so both scale alike
            g.mul_(scale * float(head.world))
            holder = ctx.w2_holder
            main = getattr(holder, "main_grad", None) if holder is not None else None
            if main is not None:
                main[head.offset: head.offset + head.shard].add_(g)
                holder.main_grad_touched = True
            else:
                dw2 = g.to(w2_shard.dtype)
        head.barrier()          # peers may reuse the slot buffers only after every rank has reduced
        return None, dh, None, dprev, dw2, None, None, None, None, None, None, None


def vocab_parallel_head_loss(head: VocabParallelHead, hidden, lm_w_shard, labels, weight, *, prev_emb=None,
                             markov_w2=None, teacher_hidden=None, t_index=None, a_ce=1.0, a_l1=0.0):
    """Sharded counterpart of ``ops.vocab_head.head_loss`` (mode 0).  ``markov_w2`` is the FULL ``[V, r]`` parameter;
    its rows of this rank's shard are used and receive gradient."""
    if teacher_hidden is not None and t_index is None:
        t_index = torch.arange(hidden.shape[0], device=hidden.device, dtype=torch.int32)
    w2_shard = head.shard_rows(markov_w2) if markov_w2 is not None else None
    holder = markov_w2 if isinstance(markov_w2, torch.nn.Parameter) else None
    return _VocabParallelLossFn.apply(
        head, hidden.contiguous(), lm_w_shard, prev_emb.contiguous() if prev_emb is not None else None,
        w2_shard.contiguous() if w2_shard is not None else None,
        teacher_hidden.contiguous() if teacher_hidden is not None else None,
        t_index.to(torch.int32).contiguous() if t_index is not None else None, labels.long().contiguous(),
        weight.float().contiguous(), float(a_ce), float(a_l1), holder)


def vocab_parallel_head_loss_reference(hidden, lm_w_shard, labels, weight, *, vocab_offset: int, group=None, prev_emb=None,
                                       markov_w2_shard=None, teacher_hidden=None, t_index=None, a_ce=1.0, a_l1=0.0):
    """Reference-math statement of the sharded head on any backend (fp32, differentiable collectives): every rank holds
    rows ``[vocab_offset, vocab_offset + V/p)`` of the head; normalisers are merged with an all-gather of the partial
    log-sum-exps, the CE target logit and the L1 partial sums with all-reduces.  Returns ``(numerator, ce, l1)`` like
    ``ops.vocab_head.head_loss_reference`` (the numerator is this rank's share: sum the ranks' numerators, or
    all-reduce gradients, exactly as for the kernel path)."""
    import torch.distributed as dist
    import torch.nn.functional as F

    from aspec_b200.parallel.cp_runtime import _AllGatherStack

    def global_lse(local_logits):
        part = torch.logsumexp(local_logits, -1)
        return torch.logsumexp(_AllGatherStack.apply(part, group), 0)

    def all_sum(x):
        return _AllGatherStack.apply(x, group).sum(0)

    logits = F.linear(hidden.float(), lm_w_shard.float())
    if prev_emb is not None:
        logits = logits + F.linear(prev_emb.float(), markov_w2_shard.float())
    lse = global_lse(logits)
    local = labels.long() - vocab_offset
    mine = (local >= 0) & (local < logits.shape[1])
    picked = logits.gather(1, local.clamp(0, logits.shape[1] - 1)[:, None])[:, 0]
    ce = lse - all_sum(torch.where(mine, picked, torch.zeros_like(picked)))
    l1 = torch.zeros_like(ce)
    if teacher_hidden is not None:
        t = F.linear(teacher_hidden.float(), lm_w_shard.float())
        if t_index is not None:
            t = t[t_index.long()]
        q = torch.exp(t - global_lse(t)[:, None])
        p = torch.exp(logits - lse[:, None])
        l1 = all_sum((p - q).abs().sum(-1))
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    num = (weight.float() * (a_ce * ce + a_l1 * l1)).sum() / world       # every rank holds the same rows
    return num, ce.detach(), l1.detach()
