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
