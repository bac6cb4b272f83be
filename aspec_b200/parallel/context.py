"""Context-parallel ownership of a sequence.

``context_shard_bounds(T, rank, world, alignment)`` is THE ownership function: with ``g = T // alignment``
aligned groups, rank ``r`` owns ``[(g * r // world) * alignment, (g * (r + 1) // world) * alignment)`` and the
last rank extends to ``T`` (reference: aspec/inference/context.py:30-55).  Packed rows apply it per document.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def context_shard_bounds(seq_len: int, rank: int, world: int, alignment: int = 1) -> Tuple[int, int]:
    if seq_len < 0 or world <= 0 or not 0 <= rank < world or alignment <= 0:
        raise ValueError("invalid context shard request")
    groups = seq_len // alignment
    start = (groups * rank // world) * alignment
    end = seq_len if rank == world - 1 else (groups * (rank + 1) // world) * alignment
    return start, end


def packed_shard_positions(document_lengths: Sequence[int], rank: int, world: int, alignment: int = 1) -> List[int]:
    """Positions of the packed row that ``rank`` owns (document-local ownership, concatenated)."""
    out: List[int] = []
    off = 0
    for n in document_lengths:
        s, e = context_shard_bounds(n, rank, world, alignment)
        out.extend(range(off + s, off + e))
        off += n
    return out
