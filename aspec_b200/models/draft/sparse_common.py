"""Shared pieces of the compressed / selected sparse-attention drafts (CSA, QSA, DSA).

Packed layout: the context is ``T`` tokens of several documents; every query row carries an interval table
``[lo, hi, b_lo, b_hi]`` whose first interval is the visible context (its document, strictly before the
anchor) and whose second is the query's own draft block in the key array.  Token groups of ``ratio`` are
aligned to the document start, so every query of a document sees the same groups
(reference: aspec/models/draft/csa.py:99-193, aspec/models/draft/qsa.py:150-280).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def rotary(values: torch.Tensor, positions: torch.Tensor, dim: int, theta: float) -> torch.Tensor:
    """Non-interleaved RoPE on ``values[..., :dim]`` (``values [N, H, d]``, ``positions [N]``)."""
    inv = theta ** (-torch.arange(0, dim, 2, device=values.device).float() / dim)
    ang = positions.float()[:, None] * inv
    cos, sin = ang.cos()[:, None], ang.sin()[:, None]
    a, b = values[..., :dim].float().chunk(2, -1)
    rot = torch.cat((a * cos - b * sin, a * sin + b * cos), -1).to(values.dtype)
    return torch.cat((rot, values[..., dim:]), -1)


@dataclass
class GroupLayout:
    """Complete ``ratio``-token groups of every document that has queries.

    ``token_index [G, ratio]`` context rows of each group, ``start``/``end [G]`` the covered range,
    ``doc [G]`` the document's first context row, ``first [G]`` true for a document's first group,
    ``position [G]`` the rotary position of the group (its first token's position).
    """
    ratio: int
    token_index: torch.Tensor
    start: torch.Tensor
    end: torch.Tensor
    doc: torch.Tensor
    first: torch.Tensor
    position: torch.Tensor

    @property
    def num_groups(self) -> int:
        return int(self.start.shape[0])


def build_group_layout(lo: torch.Tensor, hi: torch.Tensor, ctx_pos: torch.Tensor, ratio: int) -> GroupLayout:
    dev = lo.device
    lo_c, hi_c = lo.long().cpu(), hi.long().cpu()
    docs = {}
    for a, b in zip(lo_c.tolist(), hi_c.tolist()):
        docs[a] = max(docs.get(a, a), b)
    starts, doc_ids, firsts = [], [], []
    for a in sorted(docs):
        n = (docs[a] - a) // ratio
        starts += [a + g * ratio for g in range(n)]
        doc_ids += [a] * n
        firsts += [g == 0 for g in range(n)]
    start = torch.tensor(starts, dtype=torch.long, device=dev)
    token_index = start[:, None] + torch.arange(ratio, device=dev)[None]
    position = ctx_pos.long()[start] if start.numel() else start
    return GroupLayout(ratio, token_index, start, start + ratio, torch.tensor(doc_ids, dtype=torch.long, device=dev),
                       torch.tensor(firsts, dtype=torch.bool, device=dev), position)


def eligible_groups(layout: GroupLayout, lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    """``[n, G]``: the group lies in the query's document and ends at or before its anchor."""
    return (layout.doc[None] == lo.long()[:, None]) & (layout.end[None] <= hi.long()[:, None])


def masked_log_softmax(scores: torch.Tensor, mask: torch.Tensor):
    valid = mask.any(-1)
    s = scores.masked_fill(~mask, float("-inf"))
    s = torch.where(valid[:, None], s, torch.zeros_like(s))
    return torch.log_softmax(s, -1).masked_fill(~mask, 0.0), valid


def kl_rows(target: torch.Tensor, log_prob: torch.Tensor, valid: torch.Tensor) -> torch.Tensor:
    kl = (target * (torch.log(target.clamp_min(1e-20)) - log_prob)).sum(-1)
    return torch.where(valid, kl, torch.zeros_like(kl))


def gathered_attention(q, keys, values, ok, scale):
    """``q [n, H, d]`` against per-row gathered ``keys/values [n, S, Hk, d]`` with validity ``ok [n, S]``."""
    g = q.shape[1] // keys.shape[2]
    kk = keys.repeat_interleave(g, 2).float()
    vv = values.repeat_interleave(g, 2).float()
    s = torch.einsum("nhd,nshd->nhs", q.float(), kk) * scale
    s = s.masked_fill(~ok[:, None], float("-inf"))
    any_ok = ok.any(-1)[:, None, None]
    p = torch.softmax(torch.where(any_ok, s, torch.zeros_like(s)), -1)
    p = torch.where(ok[:, None], p, torch.zeros_like(p))
    return torch.einsum("nhs,nshd->nhd", p, vv).to(q.dtype)


def indexed_attention(q, keys, values, idx, ok, scale):
    """Attention of ``q [n, H, d]`` over the key rows ``idx [n, S]`` of ``keys / values [Tk, Hk, d]`` where ``ok``.

    On a GPU (bf16, head dim 128) this is the selected-key kernel: rows are gathered tile by tile inside the kernel
    and nothing of size ``n x S x Hk x d`` is materialised.  Elsewhere it is the gathered fp32 statement above."""
    from aspec_b200.ops import sparse_attention as SA
    if SA._kernel_ok(q, keys, values):
        sel = torch.where(ok, idx, torch.full_like(idx, -1)).to(torch.int32)
        out, _ = SA.selected_attention(q, keys, values, sel, scale)
        return out
    return gathered_attention(q, keys[idx], values[idx], ok, scale)


def own_block_index(iv: torch.Tensor, n_keys: int):
    b_lo, b_hi = iv[:, 2].long(), iv[:, 3].long()
    width = int((b_hi - b_lo).max().item()) if iv.shape[0] else 0
    blk = b_lo[:, None] + torch.arange(width, device=iv.device)[None]
    return blk.clamp(max=n_keys - 1), blk < b_hi[:, None]
