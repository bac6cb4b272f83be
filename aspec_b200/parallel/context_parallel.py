"""Direct context parallelism for block drafting: the context's K/V stay on the rank that owns them, queries are
read in place from their owners' memory, and partial results are written straight into the owners' memory.

Reference protocol (aspec/models/ops/direct_cp.py:287-343,460-467,1047-1100): all-gather the queries, run partial
attention against the local K/V shard, all-to-all the partial outputs and log-sum-exps back, merge.  Here the
attention kernel itself does the moving: on rank ``r`` one launch per query owner ``o`` loads ``Q_o`` by TMA from
``o``'s HBM, attends to the local K/V shard and stores the partial ``O`` / ``LSE`` into slot ``r`` of ``o``'s
buffers.  No collective moves tensor data; a stream-ordered barrier separates "partials written" from "merge".
Backward mirrors it: rank ``r`` reads ``Q_o, O_o, LSE_o, dO_o`` from the owner, keeps ``dK, dV`` of its shard local
and stores its partial ``dQ`` into slot ``r`` of the owner, who sums the slots.

Key layout on rank ``r``: ``[context rows owned by r | draft rows of r's own query blocks]``.  A query of owner
``o`` sees ``[lo, hi) ∩ [start_r, end_r)`` of the context on rank ``r`` and, only on its owner, its own block.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple

import torch

from aspec_b200.ops.attention import merge_partials
from aspec_b200.parallel.symmetric_memory import SymmetricBuffer


def _up(n: int, a: int = 256) -> int:
    return -(-n // a) * a


def local_intervals(intervals: torch.Tensor, ctx_start: int, ctx_end: int, ctx_total: int, own: bool,
                    query_start: int = 0) -> torch.Tensor:
    """Global table ``[lo, hi, b_lo, b_hi]`` (keys = ``ctx_total`` context rows then all draft rows) -> the table of the
    same queries against one rank's key array ``[ctx_start:ctx_end | own draft rows]``."""
    iv = intervals.to(torch.int64)
    a0 = iv[:, 0].clamp(ctx_start, ctx_end) - ctx_start
    a1 = iv[:, 1].clamp(ctx_start, ctx_end) - ctx_start
    a1 = torch.maximum(a0, a1)
    if own:
        shift = (ctx_end - ctx_start) - ctx_total - query_start
        b0, b1 = iv[:, 2] + shift, iv[:, 3] + shift
    else:
        b0 = b1 = torch.zeros_like(a0)
    return torch.stack([a0, a1, b0, b1], -1).to(torch.int32).contiguous()


class CPWorkspace:
    """Peer-visible buffers of one rank: its queries and results, and one slot per peer for incoming partials."""

    def __init__(self, world: int, max_queries: int, heads: int, head_dim: int, device=None,
                 buffer: Optional[SymmetricBuffer] = None):
        self.world, self.max_queries, self.heads, self.head_dim = world, max_queries, heads, head_dim
        qb = max_queries * heads * head_dim * 2
        lb = heads * max_queries * 4
        sizes = [("q", qb), ("out", qb), ("dout", qb), ("lse", lb), ("part_o", world * qb), ("part_lse", world * lb),
                 ("part_dq", world * qb)]
        self._off, off = {}, 0
        for name, n in sizes:
            self._off[name] = (off, n)
            off += _up(n)
        self.buffer = buffer if buffer is not None else SymmetricBuffer.allocate(off, device)
        raw = self.buffer.tensor
        v = lambda name, dt: raw[self._off[name][0]: self._off[name][0] + self._off[name][1]].view(dt)
        shape = (max_queries, heads, head_dim)
        self.q, self.out, self.dout = (v(n, torch.bfloat16).view(shape) for n in ("q", "out", "dout"))
        self.lse = v("lse", torch.float32)
        self.part_o = v("part_o", torch.bfloat16).view(world, *shape)
        self.part_lse = v("part_lse", torch.float32).view(world, heads * max_queries)
        self.part_dq = v("part_dq", torch.bfloat16).view(world, *shape)

    def export(self) -> dict:
        return {"memory": self.buffer.export(), "world": self.world, "max_queries": self.max_queries, "heads": self.heads,
                "head_dim": self.head_dim}

    @classmethod
    def open(cls, meta: dict) -> "CPWorkspace":
        return cls(meta["world"], meta["max_queries"], meta["heads"], meta["head_dim"], buffer=SymmetricBuffer.open(meta["memory"]))


class DirectCPAttention:
    """Phase methods (``publish -> partials -> merge`` and ``publish_grad -> grad_partials -> reduce_grad``) so that one
    process can emulate several ranks; ``barrier`` is a tiny stream-ordered collective in real runs."""

    def __init__(self, rank: int, world: int, workspaces: Sequence[CPWorkspace], barrier: Optional[Callable[[], None]] = None):
        self.rank, self.world, self.ws = rank, world, list(workspaces)
        self.mine = self.ws[rank]
        self.barrier = barrier or (lambda: None)
        self.concurrent_owners = True

    def _views(self, w: CPWorkspace, n: int):
        H = w.heads
        return w.q[:n], w.out[:n], w.dout[:n], w.lse[: H * n].view(H, n)

    # -- forward ------------------------------------------------------------------------------------------
    def publish(self, q: torch.Tensor) -> None:
        self._nq = q.shape[0]
        self.mine.q[: self._nq].copy_(q)

    def partials(self, k_local, v_local, tables: Sequence[torch.Tensor], counts: Sequence[int], scale: float) -> None:
        """``tables[o]`` / ``counts[o]``: owner ``o``'s queries against THIS rank's keys."""
        from aspec_b200.ops import attention_sm100 as K
        self._saved = (k_local, v_local, list(tables), list(counts), scale)

        def one(o: int) -> None:
            n = counts[o]
            if n == 0:
                return
            w = self.ws[o]
            H = w.heads
            K.forward(w.q[:n], k_local, v_local, tables[o], scale, out=w.part_o[self.rank, :n],
                      lse=w.part_lse[self.rank, : H * n].view(H, n))

        self._per_owner(one)

    def _per_owner(self, fn: Callable[[int], object]) -> list:
        """Run ``fn(owner)`` for every owner, each on its own CUDA stream: the owners' launches are independent (their
        queries and outputs differ, the keys are shared), and run one after another every launch would pay its own
        tail wave.  The calling stream waits for all of them; tensors returned by ``fn`` are handed over to it."""
        dev = self.mine.q.device
        if dev.type != "cuda" or self.world == 1 or not self.concurrent_owners:
            return [fn(o) for o in range(self.world)]
        cur = torch.cuda.current_stream(dev)
        if not hasattr(self, "_streams"):
            self._streams = [torch.cuda.Stream(dev) for _ in range(self.world)]
        start = cur.record_event()
        results = []
        for o, side in enumerate(self._streams):
            side.wait_event(start)
            with torch.cuda.stream(side):
                res = fn(o)
            for t in (res if isinstance(res, (tuple, list)) else (res,)):
                if torch.is_tensor(t):
                    t.record_stream(cur)
            results.append(res)
        for side in self._streams:
            cur.wait_stream(side)
        return results

    def merge(self) -> Tuple[torch.Tensor, torch.Tensor]:
        n, w = self._nq, self.mine
        H = w.heads
        out, lse = w.out[:n], w.lse[: H * n].view(H, n)
        if w.part_o.is_cuda and w.head_dim % 4 == 0:
            from aspec_b200.ops import comm
            comm.attn_merge_partials(w.part_o, w.part_lse, n, out, lse)     # one kernel, straight into the workspace
            return out.clone(), lse.clone()                                 # the workspace is reused by the next call
        merged, merged_lse = merge_partials(w.part_o[:, :n], w.part_lse[:, : H * n].view(self.world, H, n))
        out.copy_(merged)
        lse.copy_(merged_lse)
        return merged, merged_lse

    # -- backward -----------------------------------------------------------------------------------------
    def publish_grad(self, dout: torch.Tensor) -> None:
        self.mine.dout[: self._nq].copy_(dout)

    def grad_partials(self) -> Tuple[torch.Tensor, torch.Tensor]:
        from aspec_b200.ops import attention_sm100 as K
        k_local, v_local, tables, counts, scale = self._saved
        def one(o: int):
            n = counts[o]
            if n == 0:
                return None
            q, out, dout, lse = self._views(self.ws[o], n)
            if o != self.rank:
                # the dK/dV kernel re-reads the query-side tiles once per key tile: fetch the peer's rows into local
                # memory once (peer memory is not cached in this GPU's L2) and run the kernels on the copies
                q, out, dout, lse = (self._fetch(t) for t in (q, out, dout, lse))
            _dq, dk_o, dv_o = K.backward(q, k_local, v_local, tables[o], out, lse, dout, scale,
                                         dq=self.ws[o].part_dq[self.rank, :n])
            return dk_o, dv_o

        dk = torch.zeros_like(k_local, dtype=torch.float32)
        dv = torch.zeros_like(v_local, dtype=torch.float32)
        for res in self._per_owner(one):
            if res is not None:
                dk += res[0]
                dv += res[1]
        return dk.to(k_local.dtype), dv.to(v_local.dtype)

    @staticmethod
    def _fetch(peer: torch.Tensor) -> torch.Tensor:
        import ctypes as C
        from aspec_b200 import _native
        local = torch.empty(peer.shape, dtype=peer.dtype, device=peer.device)
        nbytes = peer.numel() * peer.element_size()
        rc = _native.kernels().ab_copy_bytes(C.c_void_p(peer.data_ptr()), C.c_void_p(local.data_ptr()), C.c_longlong(nbytes),
                                             C.c_void_p(torch.cuda.current_stream(peer.device).cuda_stream))
        if rc != 0:                       # sizes that are not multiples of 16 bytes take the generic copy
            local.copy_(peer)
        return local

    def reduce_grad(self) -> torch.Tensor:
        from aspec_b200.ops import comm
        n, w = self._nq, self.mine
        dq = torch.empty(n, w.heads, w.head_dim, dtype=torch.bfloat16, device=w.q.device)
        comm.peer_reduce([w.part_dq[r, :n].reshape(-1) for r in range(self.world)], dq.view(-1))
        return dq


class _DirectCPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, cp: DirectCPAttention, q, k_local, v_local, tables, counts, scale):
        cp.publish(q)
        cp.barrier()
        cp.partials(k_local, v_local, tables, counts, scale)
        cp.barrier()
        out, lse = cp.merge()
        cp.barrier()                 # merged O / LSE visible to the peers' backward
        ctx.cp = cp
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        cp = ctx.cp
        cp.publish_grad(dout.contiguous())
        cp.barrier()
        dk, dv = cp.grad_partials()
        cp.barrier()
        dq = cp.reduce_grad()
        cp.barrier()                 # slots may be overwritten by the next layer only after every owner has reduced
        return None, dq, dk, dv, None, None, None


def direct_cp_attention(cp: DirectCPAttention, q, k_local, v_local, tables, counts, scale: float):
    """``q [Q_loc, H, d]`` (this rank's queries), ``k_local / v_local [T_r + Q_loc, Hkv, d]``."""
    return _DirectCPFn.apply(cp, q.contiguous(), k_local.contiguous(), v_local.contiguous(), tables, counts, float(scale))
