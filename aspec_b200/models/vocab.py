"""Pruned Draft vocabulary.

A Draft head over a subset of the Target vocabulary is described by two tensors with the serving stack's conventions:
``t2d`` - bool ``[V_target]``, true for tokens the head predicts; ``d2t`` - int64 ``[V_draft]`` with
``target_id = draft_id + d2t[draft_id]``, head rows ordered by ascending target id
(reference: aspec/models/vocab.py:22-45).
"""
from __future__ import annotations

import hashlib

import torch


def build_vocab_mapping(selected_target_ids: torch.Tensor, target_vocab_size: int):
    """``(d2t, t2d)`` for the given target token ids (duplicates and order do not matter)."""
    kept = torch.unique(selected_target_ids.to(torch.int64))           # sorted ascending
    t2d = torch.zeros(target_vocab_size, dtype=torch.bool)
    t2d[kept] = True
    return kept - torch.arange(kept.numel()), t2d


def _mapping_problem(d2t, t2d, draft_vocab_size: int, target_vocab_size: int):
    """The first thing wrong with a mapping, or ``None``."""
    if not (torch.is_tensor(d2t) and torch.is_tensor(t2d)):
        return "d2t and t2d must be tensors"
    if (d2t.dtype, t2d.dtype) != (torch.int64, torch.bool):
        return f"expected int64 offsets and a bool membership mask, got {d2t.dtype} and {t2d.dtype}"
    if d2t.shape != (draft_vocab_size,) or t2d.shape != (target_vocab_size,):
        return (f"shapes {tuple(d2t.shape)} / {tuple(t2d.shape)} do not match a head of {draft_vocab_size} rows over "
                f"{target_vocab_size} target tokens")
    members = torch.nonzero(t2d).reshape(-1)
    if members.numel() != draft_vocab_size:
        return f"t2d marks {members.numel()} tokens, the head has {draft_vocab_size} rows"
    implied = torch.arange(draft_vocab_size, device=members.device) + d2t.to(members.device)
    if not torch.equal(implied, members):
        return "row i of the head must be the i-th marked target token (ascending ids)"
    return None


def validate_vocab_mapping(d2t, t2d, draft_vocab_size: int, target_vocab_size: int) -> None:
    problem = _mapping_problem(d2t, t2d, draft_vocab_size, target_vocab_size)
    if problem:
        raise ValueError(f"invalid vocabulary mapping: {problem}")


def vocab_mapping_manifest(d2t, t2d) -> dict:
    """Sizes, the offset convention and a digest of both tensors, for export manifests."""
    validate_vocab_mapping(d2t, t2d, d2t.numel(), t2d.numel())
    digest = hashlib.sha256()
    for tensor in (d2t, t2d):
        digest.update(tensor.detach().cpu().contiguous().numpy().tobytes())
    return {"target_vocab_size": t2d.numel(), "draft_vocab_size": d2t.numel(),
            "d2t_semantics": "target_token_id_minus_draft_token_id", "mapping_sha256": digest.hexdigest()}
