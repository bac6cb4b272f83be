"""Context-parallel runtime attached to a block-drafting wrapper (``DFlashModel.context_parallel``).

Ownership: the flattened context rows of a micro-batch are split contiguously (``context_shard_bounds``) and the kept
draft blocks are split contiguously too; a rank projects only its context rows, embeds and carries only its own blocks,
and computes the loss of its own blocks.  Attention is the only exchange: on CUDA it is
``parallel.context_parallel.direct_cp_attention`` (peer-memory queries and partial slots, one workspace per decoder
layer because a layer's buffers must survive until its backward); on CPU / gloo the same protocol runs on differentiable
all-gathers so that the wiring is testable without GPUs (reference: aspec/models/ops/direct_cp.py:287-343,460-467).
Every rank of a context-parallel group must be given the same row and the same anchors.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from aspec_b200.ops.attention import interval_attention_reference, merge_partials
from aspec_b200.parallel.context import context_shard_bounds


class _AllGatherStack(torch.autograd.Function):
    """``[p, ...]`` stack of every rank's tensor; the gradient of a rank's own slot is the sum over ranks of the
    gradients that slot received (every rank holds a copy of the stack)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.stack(parts)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[dist.get_rank(ctx.group)], None


def _pad_rows(x: torch.Tensor, n: int) -> torch.Tensor:
    if x.shape[0] == n:
        return x
    return torch.cat([x, x.new_zeros(n - x.shape[0], *x.shape[1:])])


class ContextParallel:
    def __init__(self, group=None, *, num_layers: int, max_queries: int, heads: int, head_dim: int, device=None,
                 alignment: int = 1):
        self.group = group
        self.size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.alignment, self.max_queries = alignment, max_queries
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.layers: List = []
        if self.size > 1 and self.device.type == "cuda":
            from aspec_b200.parallel.context_parallel import CPWorkspace, DirectCPAttention
            from aspec_b200.parallel.group import exchange_workspaces, make_barrier
            barrier = make_barrier(self.device, group)
            for _ in range(num_layers):
                ws = exchange_workspaces(CPWorkspace(self.size, max_queries, heads, head_dim, device=self.device),
                                         CPWorkspace.open, group=group)
                self.layers.append(DirectCPAttention(self.rank, self.size, ws, barrier))

    # -- ownership ------------------------------------------------------------------------------------------
    def context_bounds(self, n_rows: int):
        return context_shard_bounds(n_rows, self.rank, self.size, self.alignment)

    def block_bounds(self, n_blocks: int, rank: Optional[int] = None):
        per = math.ceil(n_blocks / self.size) if n_blocks else 0
        r = self.rank if rank is None else rank
        return min(r * per, n_blocks), min((r + 1) * per, n_blocks)

    # -- attention ------------------------------------------------------------------------------------------
    def attention(self, layer: int, q, k_local, v_local, tables: Sequence[torch.Tensor], counts: Sequence[int], scale: float):
        """``q [Q_loc, H, d]`` own queries; ``tables[o]`` = owner ``o``'s queries against THIS rank's keys."""
        if self.layers:
            from aspec_b200.parallel.context_parallel import direct_cp_attention
            out, _ = direct_cp_attention(self.layers[layer], q, k_local, v_local, list(tables), list(counts), scale)
            return out
        return self._collective_attention(q, k_local, v_local, tables, counts, scale)

    def _collective_attention(self, q, k_local, v_local, tables, counts, scale):
        cap = max(counts)
        q_all = _AllGatherStack.apply(_pad_rows(q, cap), self.group)                     # [p, cap, H, d]
        outs, lses = [], []
        for o in range(self.size):
            n = counts[o]
            if n == 0:
                outs.append(q.new_zeros(cap, *q.shape[1:]))
                lses.append(q.new_full((q.shape[1], cap), float("-inf"), dtype=torch.float32))
                continue
            po, pl = interval_attention_reference(q_all[o, :n], k_local, v_local, tables[o], scale)
            outs.append(_pad_rows(po, cap))
            lses.append(torch.cat([pl.float(), pl.new_full((pl.shape[0], cap - n), float("-inf"), dtype=torch.float32)], 1))
        part_o = _AllGatherStack.apply(torch.stack(outs), self.group)                    # [p(rank), p(owner), cap, H, d]
        part_l = _AllGatherStack.apply(torch.stack(lses), self.group)                    # [p(rank), p(owner), H, cap]
        mine_o, mine_l = part_o[:, self.rank, : q.shape[0]], part_l[:, self.rank, :, : q.shape[0]]
        out, _ = merge_partials(mine_o, mine_l)
        return out

    # -- teacher rows -----------------------------------------------------------------------------------------
    def gather_teacher_rows(self, flat: torch.Tensor, flat_index: torch.Tensor) -> torch.Tensor:
        """Every rank holds the full teacher tensor in this runtime (features are replicated to the group)."""
        return flat[flat_index]


def attach(model, cp: ContextParallel) -> None:
    """Give a ``DFlashModel`` / ``DSparkModel`` its context-parallel runtime."""
    model.context_parallel = cp
