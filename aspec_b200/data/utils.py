"""Collators and the run-length loss-mask codec.

* ``pack_loss_mask`` / ``unpack_loss_mask``: alternating run lengths that always start with an
  unsupervised run (possibly 0): ``[0,0,1,1,1,0,0,1,1,0] -> "2,3,2,2,1"`` (aspec/data/utils.py:359-420).
* ``DataCollatorWithPadding``: right-pads BSHD batches (aspec/data/utils.py:49).
* ``DFlashPackingCollator``: concatenates whole documents into one THD row with ``ctx_doc_ids``,
  document-local ``base_position_ids``, ``packed_document_lengths`` and, under context parallelism,
  per-document shard ownership (aspec/data/utils.py:199-356).  Overflow is an error: the controller
  owns the row and dropping a transferred document would break work accounting.
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence, Union

import torch

from aspec_b200.parallel.context import context_shard_bounds


def pack_loss_mask(mask: Union[Sequence[int], torch.Tensor]) -> str:
    values = mask.reshape(-1).tolist() if torch.is_tensor(mask) else list(mask)
    runs: List[int] = []
    current, count = 0, 0
    for v in values:
        bit = 1 if v > 0.5 else 0
        if bit == current:
            count += 1
        else:
            runs.append(count)
            current, count = bit, 1
    runs.append(count)
    return ",".join(str(r) for r in runs)


def unpack_loss_mask(packed: Union[str, Sequence[int]], length: int = None, dtype=torch.float32) -> torch.Tensor:
    runs = [int(v) for v in packed.split(",") if v] if isinstance(packed, str) else [int(v) for v in packed]
    if any(r < 0 for r in runs):
        raise ValueError("packed_loss_mask run lengths must be non-negative")
    total = sum(runs)
    length = total if length is None else int(length)
    out = torch.zeros(length, dtype=dtype)
    cursor = 0
    for i, r in enumerate(runs):
        if i % 2 == 1:
            out[cursor:min(cursor + r, length)] = 1
        cursor += r
        if cursor >= length:
            break
    return out


def last_turn_only(packed: Union[str, Sequence[int]]) -> str:
    """Keep only the final supervised run of a packed mask."""
    runs = [int(v) for v in packed.split(",") if v] if isinstance(packed, str) else list(packed)
    sup = [i for i in range(1, len(runs), 2) if runs[i] > 0]
    if not sup:
        return ",".join(str(r) for r in runs)
    last = sup[-1]
    head = sum(runs[:last])
    tail = sum(runs[last + 1:])
    out = [head, runs[last]] + ([tail] if tail else [])
    return ",".join(str(r) for r in out)


def _row(item: Dict[str, Any], name: str, length: int) -> torch.Tensor:
    value = item[name]
    if value.dim() == 1 or (name in ("hidden_states", "last_hidden_states") and value.dim() == 2):
        value = value.unsqueeze(0)
    if value.shape[0] != 1 or value.shape[1] != length:
        raise ValueError(f"packed {name} has shape {tuple(value.shape)}; expected [1, {length}, ...]")
    return value


class DataCollatorWithPadding:
    """Right-pad ``input_ids / loss_mask / hidden_states / last_hidden_states`` to the longest row."""

    def __init__(self, pad_token_id: int = 0, pad_to: int = None):
        self.pad_token_id, self.pad_to = pad_token_id, pad_to

    def __call__(self, features: List[Dict[str, Any]]) -> Dict[str, Any]:
        lens = [int(f["input_ids"].shape[-1]) for f in features]
        T = max(max(lens), self.pad_to or 0)

        def pad(t: torch.Tensor, fill) -> torch.Tensor:
            if t.dim() == 1 or (t.dim() == 2 and t.shape[0] != 1 and t.is_floating_point() and t.shape[-1] != lens[0]):
                t = t.unsqueeze(0)
            n = t.shape[1]
            if n == T:
                return t
            shape = list(t.shape)
            shape[1] = T - n
            return torch.cat([t, torch.full(shape, fill, dtype=t.dtype, device=t.device)], 1)

        batch = {
            "input_ids": torch.cat([pad(_row(f, "input_ids", n), self.pad_token_id) for f, n in zip(features, lens)]),
            "loss_mask": torch.cat([pad(_row(f, "loss_mask", n), 0) for f, n in zip(features, lens)]),
            "attention_mask": torch.cat([pad(torch.ones(1, n, dtype=torch.long), 0) for n in lens]),
        }
        for name in ("hidden_states", "last_hidden_states"):
            if all(f.get(name) is not None for f in features):
                batch[name] = torch.cat([pad(_row(f, name, n), 0) for f, n in zip(features, lens)])
        work = [f.get("_aspec_work") for f in features]
        if all(w is not None for w in work):
            batch["_aspec_work"] = work
        return batch


class DFlashPackingCollator:
    def __init__(self, max_seq_length: int, *, pad_to_max_length: bool = True, context_parallel_rank: int = 0,
                 context_parallel_size: int = 1, context_shard_alignment: int = 1):
        if max_seq_length <= 0:
            raise ValueError("DFlashPackingCollator requires max_seq_length > 0")
        self.max_seq_length = int(max_seq_length)
        self.pad_to_max_length = bool(pad_to_max_length)
        self.cp_rank, self.cp_size = int(context_parallel_rank), int(context_parallel_size)
        self.cp_alignment = int(context_shard_alignment)
        if self.cp_size <= 0 or not 0 <= self.cp_rank < self.cp_size:
            raise ValueError("Invalid packed context-parallel ownership")
        if self.cp_alignment <= 0:
            raise ValueError("Packed context shard alignment must be positive")
        if self.cp_size > 1 and self.pad_to_max_length:
            raise ValueError("Context-sharded packing requires unpadded THD rows")

    def __call__(self, features: List[Dict[str, Any]]) -> Dict[str, Any]:
        if not features:
            raise ValueError("DFlashPackingCollator received an empty row")
        lengths = [int(f["input_ids"].shape[-1]) for f in features]
        used = sum(lengths)
        if used <= 0 or used > self.max_seq_length:
            raise ValueError(f"Packed row has {used} tokens; expected 1..{self.max_seq_length}")
        pad = self.max_seq_length - used if self.pad_to_max_length else 0
        dev = features[0]["input_ids"].device

        def cat(parts, fill):
            v = torch.cat(parts, 1)
            if pad:
                shape = list(v.shape)
                shape[1] = pad
                v = torch.cat([v, torch.full(shape, fill, dtype=v.dtype, device=v.device)], 1)
            return v

        batch: Dict[str, Any] = {
            "packed_document_lengths": tuple(lengths),
            "input_ids": cat([_row(f, "input_ids", n) for f, n in zip(features, lengths)], 0),
            "attention_mask": cat([torch.ones(1, used, dtype=torch.long, device=dev)], 0),
            "loss_mask": cat([_row(f, "loss_mask", n) for f, n in zip(features, lengths)], 0),
            "ctx_doc_ids": cat([torch.full((1, n), i, dtype=torch.long, device=dev) for i, n in enumerate(lengths)], -1),
            "base_position_ids": cat([torch.arange(n, dtype=torch.long, device=dev)[None] for n in lengths], 0),
            "hidden_states": None, "last_hidden_states": None,
        }
        bounds = [context_shard_bounds(n, self.cp_rank, self.cp_size, self.cp_alignment) for n in lengths]
        for name in ("hidden_states", "last_hidden_states"):
            have = [f.get(name) is not None for f in features]
            if any(have) and not all(have):
                raise ValueError(f"{name} must be present for every packed document")
            if not all(have):
                continue
            batch[name] = cat([_row(f, name, e - s) for f, (s, e) in zip(features, bounds)], 0)
        work = [f.get("_aspec_work") for f in features]
        if not all(isinstance(w, dict) and isinstance(w.get("execution_id"), str) and w["execution_id"] for w in work):
            raise ValueError("Packed row contains incomplete work identity")
        batch["_aspec_work"] = work
        if self.cp_size > 1:
            owned, off = [], 0
            for n, (s, e) in zip(lengths, bounds):
                owned.append(torch.arange(off + s, off + e, dtype=torch.long, device=dev))
                off += n
            batch["packed_context_positions"] = torch.cat(owned)[None]
        return batch
