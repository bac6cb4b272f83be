"""Pruned draft vocabulary: ``d2t`` = target id minus draft id (int64 offsets), ``t2d`` = bool membership.
(reference: aspec/models/vocab.py:22-45)"""
from __future__ import annotations

import hashlib

import torch


def build_vocab_mapping(selected_target_ids: torch.Tensor, target_vocab_size: int):
    """From the target token ids kept in the draft head (any order) to ``(d2t, t2d)``."""
    ids = torch.unique(selected_target_ids.long()).sort().values
    t2d = torch.zeros(target_vocab_size, dtype=torch.bool)
    t2d[ids] = True
    d2t = ids - torch.arange(ids.numel())
    return d2t, t2d


def validate_vocab_mapping(d2t, t2d, draft_vocab_size: int, target_vocab_size: int) -> None:
    if not isinstance(d2t, torch.Tensor) or not isinstance(t2d, torch.Tensor):
        raise ValueError("Vocabulary mapping requires d2t and t2d tensors")
    if d2t.dtype != torch.int64 or t2d.dtype != torch.bool:
        raise ValueError("Vocabulary mapping requires int64 d2t offsets and boolean t2d membership")
    if tuple(d2t.shape) != (draft_vocab_size,) or tuple(t2d.shape) != (target_vocab_size,):
        raise ValueError("Vocabulary mapping shape does not match the configured head")
    selected = t2d.nonzero().flatten()
    if selected.numel() != draft_vocab_size or not torch.equal(
            selected, d2t.to(selected.device) + torch.arange(draft_vocab_size, device=selected.device)):
        raise ValueError("Vocabulary mapping does not bind head rows to the sorted Target tokens")


def vocab_mapping_manifest(d2t, t2d) -> dict:
    validate_vocab_mapping(d2t, t2d, d2t.numel(), t2d.numel())
    return {"target_vocab_size": t2d.numel(), "draft_vocab_size": d2t.numel(),
            "d2t_semantics": "target_token_id_minus_draft_token_id",
            "mapping_sha256": hashlib.sha256(d2t.detach().cpu().numpy().tobytes()
                                             + t2d.detach().cpu().numpy().tobytes()).hexdigest()}
