"""Row packing and loss-mask run-length helpers (Python face of ``csrc/runtime/packer.cpp``)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

from aspec_b200 import _native


@dataclass(frozen=True)
class PackingResult:
    rank_rows: List[List[int]]
    selected_indices: tuple
    packed_tokens: int
    capacity_tokens: int
    useful_anchor_starts: int

    @property
    def fill_ratio(self) -> float:
        return self.packed_tokens / self.capacity_tokens if self.capacity_tokens else 0.0


def _runs(packed_loss_mask: Union[str, Sequence[int]]):
    if isinstance(packed_loss_mask, str):
        try:
            runs = [int(v) for v in packed_loss_mask.split(",") if v]
        except ValueError:
            raise ValueError("packed_loss_mask contains a non-integer run length") from None
    else:
        runs = [int(v) for v in packed_loss_mask]
    if any(v < 0 for v in runs):
        raise ValueError("packed_loss_mask run lengths must be non-negative")
    return (C.c_longlong * len(runs))(*runs), len(runs)


def count_eligible_anchor_starts(packed_loss_mask, sample_length: int, block_size: int) -> int:
    arr, n = _runs(packed_loss_mask)
    lib = _native.runtime()
    lib.ab_count_anchor_starts.restype = C.c_longlong
    return int(lib.ab_count_anchor_starts(arr, n, C.c_longlong(sample_length), int(block_size)))


def count_eagle_supervised_positions(packed_loss_mask, sample_length: int, ttt_length: int) -> int:
    arr, n = _runs(packed_loss_mask)
    lib = _native.runtime()
    lib.ab_count_eagle_positions.restype = C.c_longlong
    return int(lib.ab_count_eagle_positions(arr, n, C.c_longlong(sample_length), int(ttt_length)))


def pack_work_aware_rows(lengths: Sequence[int], useful_work: Sequence[int], *, dp_size: int,
                         max_seq_length: int, max_selected: Optional[int] = None) -> Optional[PackingResult]:
    if len(lengths) != len(useful_work):
        raise ValueError("lengths and useful_work must have the same size")
    if dp_size <= 0 or max_seq_length <= 0:
        raise ValueError("dp_size and max_seq_length must be positive")
    if max_selected is not None and max_selected < dp_size:
        raise ValueError("max_selected must be at least dp_size")
    n = len(lengths)
    bad = [(i, v) for i, v in enumerate(lengths) if v <= 0 or v > max_seq_length]
    if bad:
        raise ValueError("Packing received work that can never fit a row: "
                         + ", ".join(f"{i}:{v}" for i, v in bad[:5]) + f"; max_seq_length={max_seq_length}")
    row_of, pos = (C.c_int * n)(), (C.c_int * n)()
    tokens, work = C.c_longlong(), C.c_longlong()
    rc = _native.runtime().ab_pack_rows(n, (C.c_int * n)(*lengths), (C.c_longlong * n)(*useful_work), int(dp_size),
                                        int(max_seq_length), -1 if max_selected is None else int(max_selected),
                                        row_of, pos, C.byref(tokens), C.byref(work))
    if rc == 1:
        return None
    if rc != 0:
        raise ValueError(f"packing failed (code {rc})")
    rows: List[List[int]] = [[] for _ in range(dp_size)]
    for i in sorted(range(n), key=lambda i: pos[i]):
        if row_of[i] >= 0:
            rows[row_of[i]].append(i)
    selected = tuple(i for i in range(n) if row_of[i] >= 0)
    return PackingResult(rows, selected, int(tokens.value), dp_size * max_seq_length, int(work.value))
