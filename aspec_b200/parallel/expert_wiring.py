"""Turns a Draft that was built with whole expert banks into an expert-parallel one for training.

``training.expert_parallel_size = ep`` splits the Draft world into groups of ``ep`` consecutive ranks.  Inside a
group every rank keeps ``E / ep`` experts of every MoE layer and tokens reach their experts through the dispatch /
combine exchange (``parallel.expert_parallel``); ranks with the same position in different groups hold replicas of
the same experts.  Tokens stay data-parallel over ALL ranks, so:

* dense parameters are reduced over the whole Draft world, as before;
* an expert's gradient already contains every token of its group that was routed to it - it is reduced only over
  the replicas of that expert (nothing at all when ``ep`` equals the world size);
* the global gradient norm adds the dense part once and the expert part of every rank of the group.

The reference has no expert parallelism (its experts are replicated: aspec/models/draft/ling_moe.py:101-115).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class ExpertParallelGroups:
    ep_rank: int
    ep_size: int
    group: Optional[dist.ProcessGroup]            # the ranks that together hold all experts (all-to-all partners)
    replica_group: Optional[dist.ProcessGroup]    # ranks holding the same experts in other groups; None if there are none
    banks: List[torch.nn.Module]


def build_groups(rank: int, world: int, ep: int):
    """Process groups for expert parallelism; every rank must call this (group creation is collective)."""
    if world % ep:
        raise ValueError("expert_parallel_size must divide the Draft world size")
    groups = [dist.new_group(list(range(g * ep, (g + 1) * ep))) for g in range(world // ep)]
    replicas = [dist.new_group(list(range(r, world, ep))) for r in range(ep)] if world > ep else [None] * ep
    return groups[rank // ep], replicas[rank % ep]


def apply_expert_parallel(model: torch.nn.Module, ep_rank: int, ep_size: int, group, replica_group=None) -> ExpertParallelGroups:
    """Shard every expert bank of ``model`` in place.  Call before the optimizer takes its views of the parameters."""
    from aspec_b200.models.draft.moe import ExpertBank
    banks = [m for m in model.modules() if isinstance(m, ExpertBank)]
    if not banks:
        raise ValueError("expert_parallel_size > 1 needs a Draft with mixture-of-experts layers")
    for bank in banks:
        bank.shard_(ep_rank, ep_size, group)
    for m in model.modules():
        if isinstance(getattr(m, "experts", None), ExpertBank):
            m.ep_group = group
    return ExpertParallelGroups(ep_rank, ep_size, group, replica_group, banks)


def attach_fused_exchange(plan: ExpertParallelGroups, max_rows: int, hidden: int, device) -> None:
    """On GPUs: peer-visible token buffers, so that dispatch / combine become the expert GEMMs' own memory traffic."""
    from aspec_b200.parallel.expert_parallel import EPWorkspace, FusedExpertParallel
    from aspec_b200.parallel.group import exchange_workspaces, make_barrier
    for bank in plan.banks:
        ws = exchange_workspaces(EPWorkspace(max_rows, hidden, device=device), EPWorkspace.open, group=plan.group)
        bank.fused_ep = FusedExpertParallel(plan.ep_rank, plan.ep_size, bank.num_experts, ws, make_barrier(device, plan.group))
