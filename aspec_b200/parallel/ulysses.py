"""Ulysses sequence<->head exchange done by the GEMMs around attention (no all-to-all collective).

Sequence-parallel attention (reference: aspec/models/ops/eagle_thd.py:32-54 ``_SequenceHeads`` and the yunchang
``SeqAllToAll4D`` calls in aspec/models/draft/llama3_eagle.py:2078-2148) needs, per layer, an all-to-all that turns
"my rows, all heads" into "all rows, my heads" for Q, K, V and the inverse for the attention output.  Here:

* sequence -> heads: the QKV projection's epilogue scatters each column block (one rank's heads) into that rank's
  receive buffer at this rank's row range - the GEMM's own stores are the all-to-all (``scatter_cols`` epilogue);
* heads -> sequence: the output projection reads its K-dimension from ``p`` sources - head group ``g`` of this rank's
  rows lives in rank ``g``'s attention output, loaded by TMA over NVLink (two sources per launch, accumulated).

The backward pass uses the same two primitives with the roles swapped.  Weight layout: the fused QKV weight's rows
are grouped per rank ``[q heads of g | k heads of g | v heads of g]`` so that a rank's columns are contiguous.
Phases are separate methods so that several ranks can be emulated in one process.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

from aspec_b200.parallel.symmetric_memory import SymmetricBuffer


def _up(n: int, a: int = 256) -> int:
    return -(-n // a) * a


def group_qkv_rows(wq, wk, wv, world: int, head_dim: int) -> torch.Tensor:
    """Reorder ``[Hq*d | Hk*d | Hk*d, D]`` projection rows into per-rank column groups."""
    hq, hk = wq.shape[0] // head_dim // world, wk.shape[0] // head_dim // world
    parts = []
    for g in range(world):
        parts += [wq[g * hq * head_dim:(g + 1) * hq * head_dim], wk[g * hk * head_dim:(g + 1) * hk * head_dim],
                  wv[g * hk * head_dim:(g + 1) * hk * head_dim]]
    return torch.cat(parts, 0).contiguous()


class UlyssesWorkspace:
    def __init__(self, world: int, rows_per_rank: int, qkv_cols: int, out_cols: int, device=None,
                 buffer: Optional[SymmetricBuffer] = None):
        """``qkv_cols`` = one rank's share of the QKV columns, ``out_cols`` = one rank's share of the attention output."""
        self.world, self.rows, self.qkv_cols, self.out_cols = world, rows_per_rank, qkv_cols, out_cols
        self.capacity = rows_per_rank
        total = world * rows_per_rank
        sizes = [("qkv", total * qkv_cols * 2), ("attn", total * out_cols * 2), ("dqkv", total * qkv_cols * 2),
                 ("dattn", total * out_cols * 2)]
        self._off, off = {}, 0
        for name, n in sizes:
            self._off[name] = (off, n)
            off += _up(n)
        self.buffer = buffer if buffer is not None else SymmetricBuffer.allocate(off, device)
        raw = self.buffer.tensor
        v = lambda name, cols: raw[self._off[name][0]: self._off[name][0] + self._off[name][1]].view(torch.bfloat16).view(total, cols)
        self.qkv, self.dqkv = v("qkv", qkv_cols), v("dqkv", qkv_cols)           # all rows, my heads
        self.attn, self.dattn = v("attn", out_cols), v("dattn", out_cols)

    def resize(self, rows: int) -> None:
        """Use the first ``world * rows`` rows of every buffer (``rows`` up to the allocated capacity)."""
        if rows > self.capacity:
            raise ValueError(f"{rows} rows per rank exceed the workspace's capacity of {self.capacity}")
        if rows == self.rows:
            return
        raw, total = self.buffer.tensor, self.world * rows
        v = lambda name, cols: raw[self._off[name][0]: self._off[name][0] + total * cols * 2].view(torch.bfloat16).view(total, cols)
        self.rows = rows
        self.qkv, self.dqkv = v("qkv", self.qkv_cols), v("dqkv", self.qkv_cols)
        self.attn, self.dattn = v("attn", self.out_cols), v("dattn", self.out_cols)

    def export(self) -> dict:
        return {"memory": self.buffer.export(), "world": self.world, "rows": self.capacity, "qkv_cols": self.qkv_cols,
                "out_cols": self.out_cols}

    @classmethod
    def open(cls, meta: dict) -> "UlyssesWorkspace":
        return cls(meta["world"], meta["rows"], meta["qkv_cols"], meta["out_cols"], buffer=SymmetricBuffer.open(meta["memory"]))


def _multi_source(sources_a: Sequence[torch.Tensor], b_full: torch.Tensor, width: int, b_t: bool = False) -> torch.Tensor:
    """``sum_g A_g @ B_g^T`` where ``A_g [M, width]`` are separate buffers and ``B_g`` is slice ``g`` of ``b_full`` along
    the reduction index (columns ``[g * width, (g + 1) * width)`` of ``[N, world * width]``, or rows of
    ``[world * width, N]`` when ``b_t``).  Two sources run as one dual-source launch of the dense kernel; more run as ONE
    grouped launch whose output tiles each reduce over ``world`` K segments inside their accumulator."""
    from aspec_b200.ops import gemm as G
    world = len(sources_a)
    piece = (lambda g: b_full[g * width:(g + 1) * width]) if b_t else (lambda g: b_full[:, g * width:(g + 1) * width])
    if world <= 2:
        a2, b2 = (sources_a[1], piece(1)) if world == 2 else (None, None)
        return G.gemm(sources_a[0], piece(0), b_t=b_t, a2=a2, b2=b2, stream_k=False)
    import numpy as np
    from aspec_b200.ops import grouped_gemm as GG
    M = sources_a[0].shape[0]
    N = b_full.shape[1] if b_t else b_full.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=b_full.device)
    m_tiles, n_tiles = -(-M // GG.BM), -(-N // GG.BN)
    total = m_tiles * n_tiles
    nt, mt = np.divmod(np.arange(total), m_tiles)
    tiles = np.zeros(total, dtype=GG._TILE)
    tiles["d"] = np.uint64(out.data_ptr()) + ((mt * GG.BM * out.stride(0) + nt * GG.BN) * 2).astype(np.uint64)
    tiles["ldd"] = out.stride(0)
    tiles["rows"] = np.minimum(GG.BM, M - mt * GG.BM)
    tiles["cols"] = np.minimum(GG.BN, N - nt * GG.BN)
    tiles["seg0"] = np.arange(total) * world
    tiles["nseg"] = world
    segs = np.zeros(total * world, dtype=GG._SEG)
    g = np.tile(np.arange(world), total)
    segs["a_map"] = g
    segs["a_mn"] = np.repeat(mt * GG.BM, world)
    segs["b_map"] = world
    segs["b_mn"] = np.repeat(nt * GG.BN, world)
    segs["b_k"] = g * width
    segs["k_blocks"] = -(-width // GG.BK)
    # a last partial k-block reads past the segment in B, but A's columns past ``width`` are the TMA zero fill
    if width % 8:
        raise ValueError("the per-rank reduction width must be a multiple of 8 elements (TMA alignment)")
    operands = [(GG._as_2d(a), 0) for a in sources_a] + [(GG._as_2d(b_full), 1)]
    GG._launch(operands, tiles, segs, False, b_t, False, 1.0, b_full.device)
    return out


class UlyssesExchange:
    def __init__(self, rank: int, world: int, workspaces: Sequence[UlyssesWorkspace], barrier: Optional[Callable[[], None]] = None):
        self.rank, self.world, self.ws = rank, world, list(workspaces)
        self.mine = self.ws[rank]
        self.barrier = barrier or (lambda: None)

    def set_rows(self, rows: int) -> None:
        """Rows per rank of the next exchange (all ranks of the group must agree)."""
        for w in self.ws:
            w.resize(int(rows))

    def _rows(self, r: int) -> slice:
        return slice(r * self.mine.rows, (r + 1) * self.mine.rows)

    def _pull(self, views: Sequence[torch.Tensor]) -> list:
        """Local copies of the peers' row blocks (this rank's own block is used in place).  The consuming GEMMs re-read
        their A rows once per column tile and peer memory is not cached in this GPU's L2, so each block crosses NVLink
        once here instead of once per tile there."""
        import ctypes as C
        from aspec_b200 import _native
        out = []
        for g, v in enumerate(views):
            if g == self.rank:
                out.append(v)
                continue
            local = torch.empty(v.shape, dtype=v.dtype, device=v.device)
            rc = _native.kernels().ab_copy_bytes(C.c_void_p(v.data_ptr()), C.c_void_p(local.data_ptr()),
                                                 C.c_longlong(v.numel() * v.element_size()),
                                                 C.c_void_p(torch.cuda.current_stream(v.device).cuda_stream))
            if rc != 0:
                raise RuntimeError(f"ab_copy_bytes refused the peer copy (code {rc})")
            out.append(local)
        return out

    # -- forward ------------------------------------------------------------------------------------------
    def project_scatter(self, x: torch.Tensor, w_grouped: torch.Tensor) -> None:
        """``x [T_loc, D] @ W^T`` with each rank's column block stored into that rank's ``qkv`` rows of this rank."""
        from aspec_b200.ops import gemm as G
        dests = [w.qkv[self._rows(self.rank)] for w in self.ws]
        G.gemm(x, w_grouped, mirrors=dests, scatter_cols=self.mine.qkv_cols)

    def received_qkv(self) -> torch.Tensor:
        return self.mine.qkv                      # [T_tot, my columns]

    def publish_attention(self, attn: torch.Tensor) -> None:
        self.mine.attn.copy_(attn.reshape(self.mine.attn.shape))

    def output_projection(self, w_o: torch.Tensor, return_rows: bool = False):
        """``out[T_loc, D] = sum_g attn_g[my rows] @ W_o[:, cols_g]^T`` with ``attn_g`` read from rank ``g``.  With
        ``return_rows`` also returns the pulled row blocks: the backward pass needs exactly these (the peers' buffers
        are overwritten by the next exchange)."""
        c = self.mine.out_cols
        rows = self._pull([w.attn[self._rows(self.rank)] for w in self.ws])
        if rows[self.rank].data_ptr() == self.mine.attn[self._rows(self.rank)].data_ptr():
            rows[self.rank] = rows[self.rank].clone() if return_rows else rows[self.rank]
        out = _multi_source(rows, w_o, c)
        return (out, rows) if return_rows else out

    # -- backward -----------------------------------------------------------------------------------------
    def output_projection_backward(self, dout: torch.Tensor, w_o: torch.Tensor, attn_rows=None):
        """``d attn_g[my rows] = dout @ W_o[:, cols_g]`` scattered to rank ``g``; returns ``dW_o`` (fp32).  ``attn_rows``:
        the blocks ``output_projection`` returned; without them the peers' buffers are read again (only valid when no
        other exchange ran in between)."""
        from aspec_b200.ops import gemm as G
        dests = [w.dattn[self._rows(self.rank)] for w in self.ws]
        G.gemm(dout, w_o, b_t=True, mirrors=dests, scatter_cols=self.mine.out_cols)
        if attn_rows is None:
            attn_rows = self._pull([w.attn[self._rows(self.rank)] for w in self.ws])
        parts = [G.gemm(dout, a, a_t=True, b_t=True, out_dtype=torch.float32, stream_k=False) for a in attn_rows]
        return torch.cat(parts, 1)                # [D, Hq*d] columns grouped by rank, as W_o's

    def received_dattn(self) -> torch.Tensor:
        return self.mine.dattn

    def publish_dqkv(self, dqkv: torch.Tensor) -> None:
        self.mine.dqkv.copy_(dqkv.reshape(self.mine.dqkv.shape))

    def projection_backward(self, x: torch.Tensor, w_grouped: torch.Tensor):
        """``dx = sum_g dqkv_g[my rows] @ W_g`` and ``dW_g = dqkv_g[my rows]^T @ x`` with ``dqkv_g`` read from rank ``g``."""
        from aspec_b200.ops import gemm as G
        c = self.mine.qkv_cols
        srcs = self._pull([w.dqkv[self._rows(self.rank)] for w in self.ws])
        dx = _multi_source(srcs, w_grouped, c, b_t=True)
        dw = torch.cat([G.gemm(s, x, a_t=True, b_t=True, out_dtype=torch.float32, stream_k=False) for s in srcs], 0)
        return dx, dw


class CollectiveUlyssesExchange:
    """The exchange's phase interface over ``torch.distributed`` collectives (any backend, any device): the reference
    statement of ``UlyssesExchange`` for CPU / gloo tests of the sequence-parallel model paths.  Every phase that moves
    data is one all-gather followed by a slice (gloo has no all-to-all)."""

    def __init__(self, rank: int, world: int, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.rows = 0
        self.barrier = lambda: None

    def set_rows(self, rows: int) -> None:
        self.rows = int(rows)

    def _rows(self, r: int) -> slice:
        return slice(r * self.rows, (r + 1) * self.rows)

    def _gather(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:                      # a ring-only group: nothing to exchange
            return x[None]
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.stack(parts)

    def _cols(self, full: torch.Tensor, width: int) -> torch.Tensor:
        """``full [world, rows, world * width]`` gathered from all sources -> this rank's column block of every source."""
        return torch.cat([full[s][:, self.rank * width:(self.rank + 1) * width] for s in range(self.world)], 0)

    def project_scatter(self, x: torch.Tensor, w_grouped: torch.Tensor) -> None:
        self.rows = x.shape[0]
        self._qkv = self._cols(self._gather(x @ w_grouped.T), w_grouped.shape[0] // self.world)

    def received_qkv(self) -> torch.Tensor:
        return self._qkv

    def publish_attention(self, attn: torch.Tensor) -> None:
        self._attn = attn.reshape(self.world * self.rows, -1)

    def output_projection(self, w_o: torch.Tensor, return_rows: bool = False):
        full = self._gather(self._attn)                                   # [world, T_tot, out_cols]
        c = full.shape[-1]
        rows = [full[g][self._rows(self.rank)] for g in range(self.world)]
        out = sum(rows[g] @ w_o[:, g * c:(g + 1) * c].T for g in range(self.world))
        return (out, rows) if return_rows else out

    def output_projection_backward(self, dout: torch.Tensor, w_o: torch.Tensor, attn_rows=None):
        c = w_o.shape[1] // self.world
        self._dattn = self._cols(self._gather(dout @ w_o), c)
        if attn_rows is None:
            full = self._gather(self._attn)
            attn_rows = [full[g][self._rows(self.rank)] for g in range(self.world)]
        return torch.cat([dout.float().T @ a.float() for a in attn_rows], 1)

    def received_dattn(self) -> torch.Tensor:
        return self._dattn

    def publish_dqkv(self, dqkv: torch.Tensor) -> None:
        self._dqkv = dqkv.reshape(self.world * self.rows, -1)

    def projection_backward(self, x: torch.Tensor, w_grouped: torch.Tensor):
        full = self._gather(self._dqkv)
        c = full.shape[-1]
        srcs = [full[g][self._rows(self.rank)] for g in range(self.world)]
        dx = sum(srcs[g] @ w_grouped[g * c:(g + 1) * c] for g in range(self.world))
        dw = torch.cat([s.float().T @ x.float() for s in srcs], 0)
        return dx, dw
