"""Sequence-parallel self-attention block over the fused Ulysses exchange.

Every rank of the group holds ``T_loc`` rows of a packed sequence.  The QKV projection's epilogue scatters each rank's
head columns straight into that rank's memory (sequence -> head all-to-all), attention runs on ``Hq / p`` query heads and
``Hkv / p`` key/value heads over all ``p * T_loc`` rows, and the output projection gathers the peers' head slices of this
rank's rows (head -> sequence all-to-all).  Backward mirrors it with the exchange's backward primitives.  The block is
an autograd function, so it drops into a decoder layer in place of ``o_proj(attention(qkv_proj(x)))``.

The reference's counterpart is the USP (Ulysses + ring) attention of its EAGLE3 Draft
(aspec/models/draft/llama3_eagle.py:1819-2151), which wraps NCCL all-to-alls around flash-attention calls.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn

from aspec_b200.parallel.ulysses import UlyssesExchange, group_qkv_rows


class _UlyssesBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_grouped, w_o, ex: UlyssesExchange, core: Callable[[torch.Tensor], torch.Tensor]):
        ex.project_scatter(x, w_grouped)
        ex.barrier()
        qkv = ex.received_qkv().detach().clone().requires_grad_(True)     # the peer-visible buffer is reused by the next layer
        with torch.enable_grad():
            attn = core(qkv)                                              # [T_tot, my head columns]
        ex.publish_attention(attn.detach())
        ex.barrier()
        out, attn_rows = ex.output_projection(w_o, return_rows=True)
        ex.barrier()                                                      # peers have read this rank's attention rows
        ctx.ex = ex
        ctx.graph = (qkv, attn, attn_rows)
        ctx.save_for_backward(x, w_grouped, w_o)
        return out

    @staticmethod
    def backward(ctx, dout):
        ex = ctx.ex
        x, w_grouped, w_o = ctx.saved_tensors
        qkv, attn, attn_rows = ctx.graph
        ex.set_rows(x.shape[0])
        d_wo = ex.output_projection_backward(dout.contiguous(), w_o, attn_rows)   # scatters d attn to the head owners
        ex.barrier()
        d_attn = ex.received_dattn().clone()
        # fills qkv.grad and the core's own parameters; the graph is retained because cores of later blocks may share
        # sub-graphs with this one (EAGLE's depth-0 keys and values are reused by every later depth)
        torch.autograd.backward(attn, d_attn.reshape(attn.shape), retain_graph=True)
        ex.publish_dqkv(qkv.grad)
        ex.barrier()
        dx, d_wg = ex.projection_backward(x, w_grouped)
        ex.barrier()
        ctx.graph = None
        return dx, d_wg.to(w_grouped.dtype), d_wo.to(w_o.dtype), None, None


def ulysses_block(x: torch.Tensor, w_grouped: torch.Tensor, w_o: torch.Tensor, ex: UlyssesExchange,
                  core: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    """``x [T_loc, D]`` -> ``[T_loc, D]``.  ``w_grouped``: QKV rows ordered rank by rank (``group_qkv_rows``); ``w_o``'s
    columns must follow the same head order (they do when heads are split contiguously); ``core(qkv)`` maps
    ``[T_tot, (hq + 2 hkv) d / p]`` to the attention output ``[T_tot, hq d / p]`` of this rank's heads."""
    return _UlyssesBlockFn.apply(x, w_grouped, w_o, ex, core)


class UlyssesSelfAttention(nn.Module):
    """GQA self-attention with interval masks (``ops.attention``), sequence-parallel over ``exchange``.

    Parameters are stored like an ordinary attention block (``q_proj / k_proj / v_proj / o_proj`` weights); the grouped
    QKV matrix is a differentiable re-ordering of them, so checkpoints are interchangeable with the single-GPU block.
    Without an exchange the module runs the same math on one GPU (the reference for its tests).
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 exchange: Optional[UlyssesExchange] = None):
        super().__init__()
        self.hq, self.hk, self.d = num_heads, num_kv_heads, head_dim
        self.q_proj = nn.Parameter(torch.empty(num_heads * head_dim, hidden_size))
        self.k_proj = nn.Parameter(torch.empty(num_kv_heads * head_dim, hidden_size))
        self.v_proj = nn.Parameter(torch.empty(num_kv_heads * head_dim, hidden_size))
        self.o_proj = nn.Parameter(torch.empty(hidden_size, num_heads * head_dim))
        for w in (self.q_proj, self.k_proj, self.v_proj, self.o_proj):
            nn.init.normal_(w, std=0.02)
        self.exchange = exchange
        self.scale = head_dim ** -0.5

    def _core(self, qkv: torch.Tensor, intervals: torch.Tensor, hq: int, hk: int) -> torch.Tensor:
        from aspec_b200.ops.attention import interval_attention
        T, d = qkv.shape[0], self.d
        q = qkv[:, : hq * d].reshape(T, hq, d)
        k = qkv[:, hq * d:(hq + hk) * d].reshape(T, hk, d)
        v = qkv[:, (hq + hk) * d:].reshape(T, hk, d)
        out, _ = interval_attention(q.contiguous(), k.contiguous(), v.contiguous(), intervals, self.scale)
        return out.reshape(T, hq * d)

    def forward(self, x: torch.Tensor, intervals_all: torch.Tensor) -> torch.Tensor:
        """``x``: this rank's rows ``[T_loc, D]``; ``intervals_all``: visible key intervals of every row of the whole
        sequence ``[T_tot, 4]`` int32 (each rank attends with all rows for its heads)."""
        ex = self.exchange
        if ex is None:
            from aspec_b200.ops.linear import linear
            qkv = torch.cat([linear(x, self.q_proj), linear(x, self.k_proj), linear(x, self.v_proj)], -1)
            return linear(self._core(qkv, intervals_all, self.hq, self.hk), self.o_proj)
        p = ex.world
        if self.hq % p or self.hk % p:
            raise ValueError("head counts must be divisible by the sequence-parallel size")
        w_grouped = group_qkv_rows(self.q_proj, self.k_proj, self.v_proj, p, self.d)
        return ulysses_block(x, w_grouped, self.o_proj, ex,
                             lambda qkv: self._core(qkv, intervals_all, self.hq // p, self.hk // p))
