"""Anchor selection for block-drafting objectives (DFlash / DSpark / DFlash2).

An *anchor* is a context position ``p`` from which the Draft predicts a block of
``block_size`` tokens.  Behaviour follows the reference sampler
(aspec/models/ops/anchors.py:31-266):

* a position is a candidate when ``p <= min(T - bs, T - 2)`` and both ``p`` and
  ``p + 1`` are supervised (and, for padded rows, inside the real document);
* row scope: with ``n`` candidates and a budget of ``A`` anchors the stride is
  ``clamp(n // A, 1, max_gap + 1)`` and one uniform phase ``o in [0, n)`` is drawn;
  slot ``i`` takes the ``((o + i * stride) mod n)``-th candidate; slots ``i >= n`` are
  marked not kept (anchor 0);
* document scope (one packed row): the same rule independently per document,
  ``min(A, len - bs + 1)`` slots each, padded to a multiple of ``alignment``;
* deterministic mode derives the generator seed from ``blake2b(seed:step:microbatch:replica)``.
"""
from __future__ import annotations

import hashlib
from typing import Optional, Sequence, Tuple

import torch


def anchor_sampling_seed(seed: int, step: int, microbatch: int, replica: int) -> int:
    key = f"{seed}:{step}:{microbatch}:{replica}".encode("ascii")
    return int.from_bytes(hashlib.blake2b(key, digest_size=8).digest(), "little") % (2 ** 63)


def candidate_mask(loss_mask: torch.Tensor, block_size: int,
                   attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Boolean ``[B, n_cand]`` where ``n_cand = min(max(T - bs, 0) + 1, T - 1)``."""
    T = loss_mask.shape[1]
    n = max(min(max(T - block_size, 0) + 1, T - 1), 0)
    ok = (loss_mask[:, :n] > 0.5) & (loss_mask[:, 1:n + 1] > 0.5)
    if attention_mask is not None:
        if attention_mask.shape != loss_mask.shape:
            raise ValueError("Anchor attention_mask and loss_mask must have identical shapes")
        am = attention_mask.bool()
        ok = ok & am[:, :n] & am[:, block_size - 1:block_size - 1 + n] & am[:, block_size:block_size + 1]
    return ok


def _pick(ordered: torch.Tensor, counts: torch.Tensor, budget: int, max_gap: int,
          u: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """ordered [R, n] ascending candidate positions (sentinels last); counts [R]; u [R] in [0,1)."""
    n = ordered.shape[1]
    safe = counts.clamp(min=1)
    stride = (counts // budget).clamp(min=1, max=max_gap + 1)
    phase = (u * safe).long()
    slot = torch.arange(budget, device=ordered.device)[None]
    rank = (phase[:, None] + slot * stride[:, None]) % safe[:, None]
    keep = slot < counts[:, None]
    chosen = ordered.gather(1, rank.clamp(max=max(n - 1, 0))) if n else torch.zeros_like(rank)
    return torch.where(keep, chosen, torch.zeros_like(chosen)), keep


def sample_anchor_positions(seq_len: int, loss_mask: torch.Tensor, num_anchors: int,
                            block_size: int, device=None, max_gap: Optional[int] = None,
                            generator: Optional[torch.Generator] = None,
                            attention_mask: Optional[torch.Tensor] = None
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row-scope sampling.  Returns ``(anchors [B, A] int64, keep [B, A] bool)``."""
    device = loss_mask.device if device is None else device
    B = loss_mask.shape[0]
    if max(seq_len - block_size, 0) == 0:
        return (torch.zeros(B, num_anchors, dtype=torch.long, device=device),
                torch.zeros(B, num_anchors, dtype=torch.bool, device=device))
    ok = candidate_mask(loss_mask, block_size, attention_mask)
    n = ok.shape[1]
    idx = torch.arange(n, device=device)[None].expand(B, -1)
    ordered = torch.where(ok, idx, torch.full_like(idx, seq_len + 1)).sort(dim=1).values
    u = torch.rand(B, device=device, generator=generator)
    return _pick(ordered, ok.sum(1), num_anchors, block_size if max_gap is None else max_gap, u)


def document_anchor_slots(document_lengths: Sequence[int], num_anchors: int, block_size: int,
                          alignment: int = 1):
    if min(num_anchors, block_size, alignment) < 1:
        raise ValueError("Anchor budget, block size and alignment must be positive")
    slots = tuple(min(num_anchors, max(n - block_size + 1, 0)) if n > block_size else 0
                  for n in document_lengths)
    total = sum(slots)
    padded = max(alignment, -(-total // alignment) * alignment)
    return slots, total, padded


def sample_document_anchor_positions(loss_mask: torch.Tensor, ctx_doc_ids: torch.Tensor,
                                     document_lengths: Sequence[int], num_anchors: int,
                                     block_size: int, generator: Optional[torch.Generator] = None,
                                     alignment: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Document-scope sampling on one packed row ``[1, T]``."""
    if loss_mask.ndim != 2 or loss_mask.shape[0] != 1 or ctx_doc_ids.shape != loss_mask.shape:
        raise ValueError("Document anchor sampling requires one packed row and aligned document IDs")
    if not document_lengths or any(n <= 0 for n in document_lengths):
        raise ValueError("Packed document lengths must be nonempty and positive")
    T = loss_mask.shape[1]
    if sum(document_lengths) > T:
        raise ValueError("Packed document lengths exceed the row")
    device = loss_mask.device
    slots, total, padded = document_anchor_slots(document_lengths, num_anchors, block_size, alignment)
    if total == 0:
        return (torch.zeros(1, padded, dtype=torch.long, device=device),
                torch.zeros(1, padded, dtype=torch.bool, device=device))
    n_docs = len(document_lengths)
    ok = candidate_mask(loss_mask, block_size)[0]
    n = ok.shape[0]
    lengths = torch.tensor(document_lengths, device=device)
    ends = lengths.cumsum(0)
    docs = ctx_doc_ids[0, :n]
    sdocs = docs.clamp(0, n_docs - 1)
    pos = torch.arange(n, device=device)
    ok = (ok & (docs >= 0) & (docs < n_docs) & (ctx_doc_ids[0, 1:n + 1] == docs)
          & (lengths[sdocs] > block_size) & (pos <= ends[sdocs] - block_size))
    counts = torch.zeros(n_docs, dtype=torch.long, device=device).scatter_add_(0, sdocs, ok.long())
    ordered = torch.where(ok, pos, torch.full_like(pos, T)).sort().values
    first = counts.cumsum(0) - counts
    safe = counts.clamp(min=1)
    stride = (counts // num_anchors).clamp(min=1, max=block_size + 1)
    phase = (torch.rand(n_docs, device=device, generator=generator) * safe).long()
    slot_t = torch.tensor(slots, device=device)
    owner = torch.repeat_interleave(torch.arange(n_docs, device=device), slot_t, output_size=total)
    local = torch.arange(total, device=device) - (slot_t.cumsum(0) - slot_t)[owner]
    rank = (phase[owner] + local * stride[owner]) % safe[owner]
    chosen = ordered[(first[owner] + rank).clamp(max=max(n - 1, 0))]
    keep = local < counts[owner]
    anchors = torch.where(keep, chosen, torch.zeros_like(chosen))
    pad = padded - total
    F = torch.nn.functional
    return F.pad(anchors, (0, pad))[None], F.pad(keep, (0, pad))[None]


def validate_injected_anchors(anchors: torch.Tensor, keep_mask: torch.Tensor, *,
                              loss_mask: torch.Tensor, num_anchors: int, block_size: int,
                              ctx_doc_ids: Optional[torch.Tensor] = None,
                              allow_partial_last_target: bool = False):
    """Checks replayed anchors before they index anything (shape, bounds, supervision, same doc)."""
    want = (loss_mask.shape[0], num_anchors)
    if tuple(anchors.shape) != want or tuple(keep_mask.shape) != want:
        raise ValueError(f"Injected anchors and keep mask must both have shape {want}")
    if anchors.dtype not in (torch.int32, torch.int64) or keep_mask.dtype != torch.bool:
        raise ValueError("Injected anchors must be integer and keep mask must be boolean")
    anchors = anchors.to(loss_mask.device, torch.long)
    keep_mask = keep_mask.to(loss_mask.device)
    anchors = torch.where(keep_mask, anchors, torch.zeros_like(anchors))
    T = loss_mask.shape[1]
    if ((anchors < 0) | (anchors >= max(T - 1, 0)))[keep_mask].any():
        raise ValueError("Kept injected anchors must have an in-bounds first prediction target")
    if not keep_mask.any():
        return anchors, keep_mask
    nxt = (anchors + 1).clamp(max=T - 1)
    good = (loss_mask.gather(1, anchors) > 0.5) & (loss_mask.gather(1, nxt) > 0.5)
    if not good[keep_mask].all():
        raise ValueError("Kept injected anchors and their first targets must be supervised")
    if ctx_doc_ids is not None:
        if ctx_doc_ids.shape != loss_mask.shape:
            raise ValueError("ctx_doc_ids and loss_mask must have identical shapes")
        docs = ctx_doc_ids.to(loss_mask.device)
        last = (anchors + block_size - int(allow_partial_last_target)).clamp(max=T - 1)
        a_doc = docs.gather(1, anchors)
        same = (a_doc >= 0) & (a_doc == docs.gather(1, last))
        if not same[keep_mask].all():
            raise ValueError("Kept injected anchor blocks must not cross document boundaries")
    return anchors, keep_mask
