"""Assistant-span loss mask on token ids (native scan in ``csrc/runtime/packer.cpp``): tokens between an assistant
header and the end-of-turn marker are supervised (reference: aspec/models/ops/loss_mask.py:26-115)."""
from __future__ import annotations

import ctypes as C
from typing import Sequence, Tuple

import torch

from aspec_b200 import _native


def compute_assistant_loss_mask(input_ids: torch.Tensor, header_ids: Sequence[int], end_ids: Sequence[int],
                                skip_after_header: int = 0, last_turn_only: bool = False) -> Tuple[torch.Tensor, int]:
    """Returns ``(mask [T] uint8, start of the last assistant span)``."""
    ids = input_ids.reshape(-1).to(torch.int64).contiguous().cpu()
    n = ids.numel()
    out = torch.zeros(n, dtype=torch.uint8)
    header = (C.c_longlong * max(len(header_ids), 1))(*header_ids)
    end = (C.c_longlong * max(len(end_ids), 1))(*end_ids)
    lib = _native.runtime()
    lib.ab_assistant_loss_mask.restype = C.c_longlong
    last = lib.ab_assistant_loss_mask(C.c_void_p(ids.data_ptr()), C.c_longlong(n), header, len(header_ids), end,
                                      len(end_ids), int(skip_after_header), C.c_void_p(out.data_ptr()))
    if last_turn_only and n:
        out[:last] = 0
    return out, int(last)
