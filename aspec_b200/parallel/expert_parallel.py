"""Expert parallelism: all-to-all dispatch of expert-sorted tokens, local expert GEMMs, all-to-all combine.

The reference replicates every expert on every rank (aspec/models/draft/ling_moe.py:101-115); expert
parallelism is new here.  Tokens arrive sorted by global expert id, so the rows bound for rank ``r`` are one
contiguous slice; counts are exchanged first, then the rows (``all_to_all_single`` with uneven splits, which
autograd reverses for the backward), the local bank runs one GEMM per expert, and the results return along
the same route.  ``all_to_all_single`` over NCCL is the measured baseline of this path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty(sum(out_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        gx = g.new_empty(sum(ctx.in_splits), *g.shape[1:])
        dist.all_to_all_single(gx, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return gx, None, None, None


def dispatch_combine(bank, x_sorted: torch.Tensor, sorted_expert: torch.Tensor, group=None) -> torch.Tensor:
    ep = bank.ep_size
    E_local = bank.local_experts
    counts = torch.bincount(sorted_expert, minlength=bank.num_experts)            # per global expert
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)                        # [ep * E_local]: from each rank
    send_splits = counts.view(ep, E_local).sum(1).tolist()
    recv_matrix = recv_counts.view(ep, E_local)
    recv_splits = recv_matrix.sum(1).tolist()
    recv = _AllToAll.apply(x_sorted, recv_splits, send_splits, group)
    # received rows are grouped (source rank, local expert); regroup by local expert for the bank
    src_rank = torch.repeat_interleave(torch.arange(ep, device=recv.device), torch.tensor(recv_splits, device=recv.device))
    local_expert = torch.repeat_interleave(torch.arange(E_local, device=recv.device).repeat(ep), recv_matrix.reshape(-1))
    order = torch.argsort(local_expert, stable=True)
    y = bank(recv[order], recv_matrix.sum(0).tolist())
    back = torch.empty_like(y)
    back[order] = y
    return _AllToAll.apply(back, send_splits, recv_splits, group)


# ---------------------------------------------------------------------------------------------------------------
# Fused dispatch / combine over peer memory
# ---------------------------------------------------------------------------------------------------------------
class EPWorkspace:
    """Peer-visible buffers of one rank: its expert-sorted tokens (``x``), the rows returned by the experts (``y``) and
    the same pair for the backward pass (``dy`` sent to the experts, ``dx`` returned)."""

    def __init__(self, max_rows: int, hidden: int, device=None, buffer=None):
        from aspec_b200.parallel.symmetric_memory import SymmetricBuffer
        self.max_rows, self.hidden = max_rows, hidden
        n = max_rows * hidden * 2
        n = -(-n // 256) * 256
        self.buffer = buffer if buffer is not None else SymmetricBuffer.allocate(4 * n, device)
        raw = self.buffer.tensor
        if buffer is None:
            raw.zero_()          # rows past a run's end are read (and masked or multiplied by zero): keep them finite
        view = lambda i: raw[i * n: i * n + max_rows * hidden * 2].view(torch.bfloat16).view(max_rows, hidden)
        self.x, self.y, self.dy, self.dx = view(0), view(1), view(2), view(3)

    def export(self) -> dict:
        return {"memory": self.buffer.export(), "max_rows": self.max_rows, "hidden": self.hidden}

    @classmethod
    def open(cls, meta: dict) -> "EPWorkspace":
        from aspec_b200.parallel.symmetric_memory import SymmetricBuffer
        return cls(meta["max_rows"], meta["hidden"], buffer=SymmetricBuffer.open(meta["memory"]))


class FusedExpertParallel:
    """Expert-parallel MoE whose all-to-alls are the expert GEMMs' own memory traffic.

    Every rank sorts its routed tokens by global expert into its peer-visible ``x``.  The owner of expert ``e`` pulls
    the rows bound for it from every source's ``x`` once (the dispatch: each row crosses NVLink exactly once, no
    split-size negotiation beyond the count matrix, no collective) and its down GEMM stores its output straight into
    the source's ``y`` (the combine: the transfer is the epilogue's own stores, tile by tile).  All (source, expert) pairs of a
    phase run as one grouped launch (``ops/grouped_gemm.py``).  Only the ``[ranks, experts]`` count
    matrix is exchanged beforehand (the same host-side split sizes the all-to-all baseline needs).
    The backward pass mirrors it: ``dy`` rows are pulled from the source, ``dx`` rows are pushed back, weight gradients
    stay local.  Phases are separate methods so several ranks can be emulated in one process.
    """

    def __init__(self, rank: int, world: int, num_experts: int, workspaces, barrier=None):
        if num_experts % world:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        self.rank, self.world, self.E = rank, world, num_experts
        self.local = num_experts // world
        self.ws = list(workspaces)
        self.mine = self.ws[rank]
        self.barrier = barrier or (lambda: None)

    # -- forward ------------------------------------------------------------------------------------------
    def publish(self, x_sorted: torch.Tensor) -> None:
        self._n = x_sorted.shape[0]
        self.mine.x[: self._n].copy_(x_sorted)

    def _problems(self, count_matrix):
        """Runs of rows this rank's experts own, as parallel arrays: source rank, local expert, row offset inside the
        source's run for this rank, row count, row offset in this rank's padded staging layout; plus every source's
        ``(first row, row count)`` of that run in its sorted buffer (this rank's experts are adjacent there)."""
        import numpy as np
        from aspec_b200.ops.grouped_gemm import padded_offsets
        counts = np.asarray(count_matrix, dtype=np.int64)                    # [ranks, experts]
        offs = np.cumsum(counts, 1) - counts
        mine = slice(self.rank * self.local, (self.rank + 1) * self.local)
        src = np.repeat(np.arange(self.world), self.local)
        le = np.tile(np.arange(self.local), self.world)
        rows = counts[:, mine].reshape(-1)
        span0 = offs[:, self.rank * self.local]
        span = counts[:, mine].sum(1)
        row0 = (offs[:, mine] - span0[:, None]).reshape(-1)
        pstart, ptotal = padded_offsets(rows)
        return src, le, row0, rows, pstart, ptotal, span0, span

    def _pull(self, bufs, span0, span):
        """Bring every source's rows for this rank's experts into local memory, once: a GEMM re-reads its A rows for
        every column tile, and peer memory is not cached in this GPU's L2, so reading them in place would cross NVLink
        once per column tile.  The rank's own rows are used where they are."""
        import ctypes as C
        from aspec_b200 import _native
        out = []
        for s, buf in enumerate(bufs):
            view = buf[int(span0[s]): int(span0[s] + span[s])]
            if s == self.rank or view.shape[0] == 0:
                out.append(view if view.shape[0] else buf[:1])
                continue
            local = torch.empty(view.shape, dtype=view.dtype, device=view.device)
            rc = _native.kernels().ab_copy_bytes(C.c_void_p(view.data_ptr()), C.c_void_p(local.data_ptr()),
                                                 C.c_longlong(view.numel() * view.element_size()),
                                                 C.c_void_p(torch.cuda.current_stream(view.device).cuda_stream))
            if rc != 0:
                raise RuntimeError(f"ab_copy_bytes refused the peer copy (code {rc})")
            out.append(local)
        return out

    def run_experts(self, count_matrix, gate_up: torch.Tensor, down: torch.Tensor, clamp: float = 0.0) -> None:
        """``count_matrix[s][e]``: rows rank ``s`` routed to global expert ``e`` (host ints).  ``gate_up [E_local, 2I, D]``,
        ``down [E_local, D, I]``.  The dispatch is one pull of each source's rows; the gate/up GEMM is one grouped
        launch over all (source, expert) pairs; the down GEMM, again one grouped launch, stores its rows straight into
        every source rank's ``y`` (the combine).  Keeps the activations needed by the backward pass."""
        import numpy as np
        from aspec_b200.ops.activation import swiglu
        from aspec_b200.ops.grouped_gemm import rows_gemm
        src, le, row0, rows, pstart, ptotal, span0, span = self._problems(count_matrix)
        zeros = np.zeros_like(src)
        if ptotal == 0:                  # nothing routed here: the peers' y rows come from the other expert owners
            self._saved = (src, le, row0, rows, pstart, ptotal, span0, span, None, None, None)
            return
        xs = self._pull([w.x for w in self.ws], span0, span)
        gu = torch.zeros(ptotal, gate_up.shape[1], dtype=gate_up.dtype, device=gate_up.device)
        rows_gemm(xs, gate_up, [gu], src=src, a_row=row0, rows=rows, expert=le, dst=zeros, out_row=pstart)
        act = swiglu(gu, clamp)
        rows_gemm([act], down, [w.y for w in self.ws], src=zeros, a_row=pstart, rows=rows, expert=le, dst=src,
                  out_row=row0 + span0[src])
        self._saved = (src, le, row0, rows, pstart, ptotal, span0, span, xs, gu, act)

    def collect(self) -> torch.Tensor:
        return self.mine.y[: self._n]

    # -- backward -----------------------------------------------------------------------------------------
    def publish_grad(self, dy_sorted: torch.Tensor) -> None:
        self.mine.dy[: self._n].copy_(dy_sorted)

    def run_experts_backward(self, gate_up: torch.Tensor, down: torch.Tensor, clamp: float = 0.0):
        """Returns ``(d gate_up, d down)`` of the local experts (fp32); pushes ``dx`` rows back to their sources.
        ``dy`` rows are pulled once; five grouped launches follow: weight gradients reduce over every source's rows
        inside one accumulator per output tile, ``dx`` rows are stored into the sources' buffers."""
        import numpy as np
        from aspec_b200.ops.activation import swiglu_backward
        from aspec_b200.ops.grouped_gemm import rows_gemm, wgrad_gemm
        src, le, row0, rows, pstart, ptotal, span0, span, xs, gu, act = self._saved
        if ptotal == 0:                  # no token of any rank chose this rank's experts in this micro-batch
            self._saved = None
            return (torch.zeros(gate_up.shape, dtype=torch.float32, device=gate_up.device),
                    torch.zeros(down.shape, dtype=torch.float32, device=down.device))
        zeros = np.zeros_like(src)
        dys = self._pull([w.dy for w in self.ws], span0, span)
        d_act = torch.zeros(ptotal, down.shape[2], dtype=down.dtype, device=down.device)
        rows_gemm(dys, down, [d_act], src=src, a_row=row0, rows=rows, expert=le, dst=zeros, out_row=pstart, b_t=True)
        d_gu_rows = swiglu_backward(gu, d_act, clamp)                              # zero padding rows stay zero
        d_dn = torch.empty(down.shape, dtype=torch.float32, device=down.device)
        wgrad_gemm(dys, [act], d_dn, expert=le, a_src=src, a_row=row0, b_src=zeros, b_row=pstart, rows=rows)
        d_gu = torch.empty(gate_up.shape, dtype=torch.float32, device=gate_up.device)
        wgrad_gemm([d_gu_rows], xs, d_gu, expert=le, a_src=zeros, a_row=pstart, b_src=src, b_row=row0, rows=rows)
        rows_gemm([d_gu_rows], gate_up, [w.dx for w in self.ws], src=zeros, a_row=pstart, rows=rows, expert=le, dst=src,
                  out_row=row0 + span0[src], b_t=True)
        self._saved = None
        return d_gu, d_dn

    def collect_grad(self) -> torch.Tensor:
        return self.mine.dx[: self._n]


class _FusedEPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ep: FusedExpertParallel, x_sorted, gate_up, down, count_matrix, clamp):
        ep.publish(x_sorted)
        ep.barrier()
        ep.run_experts(count_matrix, gate_up, down, clamp)
        ep.barrier()
        y = ep.collect().clone()
        ctx.ep, ctx.clamp = ep, clamp
        ctx.save_for_backward(gate_up, down)
        return y

    @staticmethod
    def backward(ctx, dy):
        ep = ctx.ep
        gate_up, down = ctx.saved_tensors
        ep.publish_grad(dy.contiguous())
        ep.barrier()
        d_gu, d_dn = ep.run_experts_backward(gate_up, down, ctx.clamp)
        ep.barrier()
        dx = ep.collect_grad().clone()
        ep.barrier()                      # the next layer may overwrite x / dy only after every expert owner has read them
        return None, dx, d_gu.to(gate_up.dtype), d_dn.to(down.dtype), None, None


def exchange_counts(sorted_expert: torch.Tensor, num_experts: int, group=None):
    """``[ranks][experts]`` routed-row counts of every rank (one small all-gather and one host read)."""
    counts = torch.bincount(sorted_expert, minlength=num_experts)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return [counts.tolist()]
    allc = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(allc, counts, group=group)
    return torch.stack(allc).tolist()


def fused_dispatch_combine(ep: FusedExpertParallel, bank, x_sorted: torch.Tensor, sorted_expert: torch.Tensor, group=None):
    """Drop-in for ``dispatch_combine`` on CUDA bf16: same inputs, the expert bank's stacked weights are used directly."""
    counts = exchange_counts(sorted_expert, bank.num_experts, group)
    return _FusedEPFn.apply(ep, x_sorted.contiguous(), bank.gate_up_proj, bank.down_proj, counts, float(bank.clamp))
