"""Interval-masked attention over packed (THD) tokens.

Every Draft attention pattern in this framework reduces to: query row ``i`` sees the
keys in ``[a0_i, a1_i) U [b0_i, b1_i)`` of one flat key/value array.  For block
drafting the first interval is the visible context prefix of the row's anchor
(document start or window start up to, not including, the anchor) and the second
is the row's own draft block (whole block when bidirectional, up to the row's own
slot when causal).  This is the "5-endpoint" interval form of the reference
(aspec/models/ops/cudnn_flex_attention.py:53-170); the visibility rule itself is
aspec/models/dflash.py:71-131 and aspec/models/ops/direct_cp.py:382-425.

``interval_attention`` runs the hand-written sm_100a kernels on CUDA tensors and
the fp32 dense-mask reference on CPU tensors.  The reference is also the oracle
the kernel tests compare against.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

MASK_VALUE = float("-inf")


def build_block_intervals(anchors: torch.Tensor, keep: torch.Tensor, *, ctx_len: int,
                          block_size: int, doc_start: Optional[torch.Tensor] = None,
                          context_window: Optional[int] = None,
                          query_window: Optional[int] = None, causal: bool = False,
                          ctx_offset: int = 0, draft_offset: Optional[int] = None,
                          block_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Intervals ``[n_blocks * block_size, 4]`` (int32) for one packed row.

    ``anchors`` / ``keep``: ``[n_blocks]``.  Keys are laid out as ``ctx_len`` context tokens
    (starting at ``ctx_offset``) followed by the draft blocks (starting at ``draft_offset``,
    default ``ctx_offset + ctx_len``), block ``block_index[i]`` (default ``i``) occupying
    ``block_size`` consecutive slots.  ``doc_start[i]`` is the first context position of the
    anchor's document (0 when not packed).  ``context_window`` limits the prefix to the last
    ``w`` tokens before the anchor (anchor-context semantics); ``query_window`` applies the
    query-relative window ``(p + j) - key < w`` and ``|j - j'| < w`` inside the block.
    Rows of blocks that are not kept get empty intervals.
    """
    n = anchors.shape[0]
    dev = anchors.device
    j = torch.arange(block_size, device=dev)[None]                    # [1, bs]
    p = anchors.long()[:, None]                                       # [n, 1]
    lo = torch.zeros_like(p) if doc_start is None else doc_start.long()[:, None]
    if context_window is not None:
        lo = torch.maximum(lo, p - context_window)
    lo = lo.expand(n, block_size)
    hi = p.expand(n, block_size)
    if query_window is not None:
        lo = torch.maximum(lo, p + j - query_window + 1)
    lo = torch.minimum(lo, hi)
    if draft_offset is None:
        draft_offset = ctx_offset + ctx_len
    bidx = torch.arange(n, device=dev) if block_index is None else block_index.long()
    base = (draft_offset + bidx * block_size)[:, None]
    b_lo = base.expand(n, block_size).clone()
    b_hi = (base + block_size).expand(n, block_size).clone()
    if causal:
        b_hi = base + j + 1
    if query_window is not None:
        b_lo = torch.maximum(b_lo, base + j - query_window + 1)
        b_hi = torch.minimum(b_hi, base + j + query_window)
    out = torch.stack([lo + ctx_offset, hi + ctx_offset, b_lo, b_hi], dim=-1)
    out = torch.where(keep.bool()[:, None, None], out, torch.zeros_like(out))
    return out.reshape(n * block_size, 4).to(torch.int32)


def dense_interval_mask(intervals: torch.Tensor, n_keys: int) -> torch.Tensor:
    """Boolean ``[Q, n_keys]`` visibility matrix of an interval table."""
    k = torch.arange(n_keys, device=intervals.device)[None]
    iv = intervals.long()
    return ((k >= iv[:, 0:1]) & (k < iv[:, 1:2])) | ((k >= iv[:, 2:3]) & (k < iv[:, 3:4]))


def interval_attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                 intervals: torch.Tensor, scale: Optional[float] = None
                                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 (or fp64) dense-mask attention.  ``q [Q,Hq,d]``, ``k [Tk,Hkv,d]``, ``v [Tk,Hkv,dv]``.

    Returns ``out [Q,Hq,dv]`` (input dtype) and ``lse [Hq,Q]`` in the statistics dtype.  Rows
    with no visible key give zero output and ``lse = -inf``.
    """
    Q, Hq, d = q.shape
    Hkv = k.shape[1]
    if Hq % Hkv:
        raise ValueError("query heads must be a multiple of key/value heads")
    g = Hq // Hkv
    st = torch.float64 if q.dtype == torch.float64 else torch.float32
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    qf = q.to(st).transpose(0, 1)                                   # [Hq,Q,d]
    kf = k.to(st).transpose(0, 1).repeat_interleave(g, 0)          # [Hq,Tk,d]
    vf = v.to(st).transpose(0, 1).repeat_interleave(g, 0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    vis = dense_interval_mask(intervals, k.shape[0])[None]
    s = s.masked_fill(~vis, MASK_VALUE)
    lse = torch.logsumexp(s, dim=-1)
    has = torch.isfinite(lse)
    p = torch.exp(s - torch.where(has, lse, torch.zeros_like(lse))[..., None])
    p = torch.where(has[..., None], p, torch.zeros_like(p))
    out = torch.matmul(p, vf).transpose(0, 1).to(q.dtype)
    return out.contiguous(), lse


def merge_partials(outputs: torch.Tensor, lses: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact merge of attention partials over disjoint key sets.

    ``outputs [P, Q, H, dv]``, ``lses [P, H, Q]``.  Rows where no part saw a key give zero output
    and ``lse = -inf`` (reference: aspec/models/ops/direct_cp.py:460-467).
    """
    has = torch.isfinite(lses).any(0)
    safe = torch.where(has[None], lses, torch.zeros_like(lses))
    lse = torch.logsumexp(safe, dim=0)
    w = torch.exp(lses - lse[None])
    w = torch.where(has[None], w, torch.zeros_like(w))
    out = (w.permute(0, 2, 1)[..., None] * outputs.to(w.dtype)).sum(0)
    return out.to(outputs.dtype), torch.where(has, lse, torch.full_like(lse, MASK_VALUE))


class _IntervalAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, intervals, scale):
        from aspec_b200.ops import attention_sm100 as K
        out, lse = K.forward(q, k, v, intervals, scale)
        ctx.save_for_backward(q, k, v, intervals, out, lse)
        ctx.scale = scale
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        from aspec_b200.ops import attention_sm100 as K
        q, k, v, intervals, out, lse = ctx.saved_tensors
        dq, dk, dv = K.backward(q, k, v, intervals, out, lse, dout.contiguous(), ctx.scale)
        return dq, dk, dv, None, None


def _group_split(hq: int, hkv: int):
    """Widths (each one the kernels tile: 16, 8, 4, 2, 1) that add up to the query heads per key head, or ``None``."""
    if hkv <= 0 or hq % hkv:
        return None
    g, parts = hq // hkv, []
    if g in (1, 2, 4, 8, 16) or g > 31:
        return None
    for width in (16, 8, 4, 2, 1):
        while g >= width:
            parts.append(width)
            g -= width
    return parts


def interval_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, intervals: torch.Tensor,
                       scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Differentiable interval attention: tcgen05 kernels on CUDA, fp32 reference on CPU."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    from aspec_b200.ops.observed import note
    if q.is_cuda:
        from aspec_b200.ops import attention_sm100 as K
        if K.supported(q, k, v):
            note("attention", "tcgen05_interval_flash")
            return _IntervalAttentionFn.apply(q.contiguous(), k.contiguous(), v.contiguous(),
                                              intervals.contiguous(), scale)
        parts = _group_split(q.shape[1], k.shape[1])
        if parts is not None and K.supported(q[:, : k.shape[1]], k, v):
            # a query-head group the kernels do not tile (5, 6, 10, ...) is cut into groups they do (4 + 1, 4 + 2, 8 + 2):
            # one launch per piece over the same keys; autograd sums the pieces' key / value gradients
            note("attention", "tcgen05_interval_flash")
            hkv, g = k.shape[1], q.shape[1] // k.shape[1]
            qg = q.reshape(q.shape[0], hkv, g, q.shape[-1])
            outs, lses, at = [], [], 0
            kc, vc, ivc = k.contiguous(), v.contiguous(), intervals.contiguous()
            for width in parts:
                piece = qg[:, :, at:at + width].reshape(q.shape[0], hkv * width, q.shape[-1]).contiguous()
                o, l = _IntervalAttentionFn.apply(piece, kc, vc, ivc, scale)
                outs.append(o.reshape(q.shape[0], hkv, width, v.shape[-1]))
                lses.append(l.reshape(hkv, width, q.shape[0]))
                at += width
            return (torch.cat(outs, 2).reshape(q.shape[0], q.shape[1], v.shape[-1]),
                    torch.cat(lses, 1).reshape(q.shape[1], q.shape[0]))
        note("attention", "dense_mask_fp32")
        return K.unsupported_shape_fallback(q, k, v, intervals, scale)
    note("attention", "reference_fp32_cpu")
    return interval_attention_reference(q, k, v, intervals, scale)
