"""Helpers shared by the peer-memory parallel layers: workspace exchange inside a process group and the
stream-ordered barrier that separates "peers have written" from "I read"."""
from __future__ import annotations

from typing import Callable, List

import torch
import torch.distributed as dist


def exchange_workspaces(local, open_fn: Callable[[dict], object], group=None) -> List:
    """Every rank exports its workspace once per importer and opens every peer's.  Returns the list indexed by rank
    (the local object at this rank's index).  CUDA IPC handles are opened with the importing GPU current."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    mine = [local.export() for _ in range(world)]
    gathered: List = [None] * world
    dist.all_gather_object(gathered, mine, group=group)
    return [local if r == rank else open_fn(gathered[r][rank]) for r in range(world)]


def make_barrier(device, group=None) -> Callable[[], None]:
    """A tiny all-reduce on the current stream: kernels queued after it run after every peer's kernels queued before
    theirs (no host synchronisation)."""
    token = torch.zeros(1, device=device)

    def barrier() -> None:
        dist.all_reduce(token, group=group)

    return barrier
