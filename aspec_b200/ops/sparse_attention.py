"""Selected-key attention, lightning-indexer scores and top-k selection.

On a B200 these are the kernels of ``csrc/sparse_attention_sm100.cu`` and ``csrc/indexer_sm100.cu``; the PyTorch
statements in this file are their fp32 oracles and the CPU path.  They replace what the reference builds from
flash-attention varlen calls over compacted key lists, an ``einsum`` + ReLU + weighted head sum, and ``torch.topk``
(aspec/models/ops/compact_varlen.py:27-176, aspec/models/draft/dsa.py:163-205,385-418).

* :func:`selected_attention` - every query attends its own list of key rows ``sel [n, L]`` (negative = empty slot);
  differentiable in ``q``, ``keys`` and ``values``.
* :func:`indexer_scores` - ``score[q, t] = sum_h w[q, h] relu(qi[q, h] . ki[t])`` on ``[lo_q, hi_q)``, ``-inf`` elsewhere
  (selection only: no gradient; the KL terms recompute the few scores they need).
* :func:`topk_select` - indices of the ``k`` best eligible keys per row, ascending, ``-1`` padded.
"""
from __future__ import annotations

import ctypes as _c
import math
from typing import Optional, Tuple

import torch

from aspec_b200.ops.observed import note

HEAD_DIM = 128
MAX_GROUP = 16


# ------------------------------------------------------------------------------------------ oracles ----
def selected_attention_reference(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, sel: torch.Tensor,
                                 scale: float, chunk_rows: int = 256) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 statement: ``q [n, Hq, d]``, ``keys / values [Tk, Hkv, d]``, ``sel [n, L]``.  Returns ``(out, lse [Hq, n])``."""
    n, hq, _ = q.shape
    hkv = keys.shape[1]
    g = hq // hkv
    outs, lses = [], []
    for lo in range(0, max(n, 1), chunk_rows):
        s_idx = sel[lo:lo + chunk_rows].long()
        if s_idx.shape[0] == 0:
            break
        ok = (s_idx >= 0) & (s_idx < keys.shape[0])
        safe = s_idx.clamp(0, max(keys.shape[0] - 1, 0))
        kk = keys[safe].float().repeat_interleave(g, 2)                   # [c, L, Hq, d]
        vv = values[safe].float().repeat_interleave(g, 2)
        s = torch.einsum("nhd,nlhd->nhl", q[lo:lo + chunk_rows].float(), kk) * scale
        s = s.masked_fill(~ok[:, None], float("-inf"))
        lse = torch.logsumexp(s, -1)
        has = torch.isfinite(lse)
        p = torch.exp(s - torch.where(has, lse, torch.zeros_like(lse))[..., None])
        p = torch.where(has[..., None] & ok[:, None], p, torch.zeros_like(p))
        outs.append(torch.einsum("nhl,nlhd->nhd", p, vv))
        lses.append(torch.where(has, lse, torch.full_like(lse, float("-inf"))))
    if not outs:
        return q.new_zeros(q.shape), q.new_full((hq, 0), float("-inf"), dtype=torch.float32)
    return torch.cat(outs).to(q.dtype), torch.cat(lses).t().contiguous()


def indexer_scores_reference(qi: torch.Tensor, ki: torch.Tensor, w: torch.Tensor, lo: torch.Tensor,
                             hi: torch.Tensor) -> torch.Tensor:
    s = (torch.einsum("nhd,td->nht", qi.float(), ki.float()).relu_() * w.float()[:, :, None]).sum(1)
    t = torch.arange(ki.shape[0], device=qi.device)[None]
    return s.masked_fill(~((t >= lo[:, None]) & (t < hi[:, None])), float("-inf"))


def topk_select_reference(scores: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, k: int) -> torch.Tensor:
    n, T = scores.shape
    t = torch.arange(T, device=scores.device)[None]
    masked = scores.float().masked_fill(~((t >= lo[:, None]) & (t < hi[:, None])), float("-inf"))
    kk = min(k, T)
    top = masked.topk(kk, -1)
    idx = torch.where(torch.isfinite(top.values), top.indices, torch.full_like(top.indices, T + 1))
    idx = idx.sort(-1).values
    idx = torch.where(idx > T, torch.full_like(idx, -1), idx)
    if kk < k:
        idx = torch.nn.functional.pad(idx, (0, k - kk), value=-1)
    return idx.to(torch.int32)


# ------------------------------------------------------------------------------------------ kernels ----
def _kernel_ok(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor) -> bool:
    if not (q.is_cuda and q.dtype == keys.dtype == values.dtype == torch.bfloat16):
        return False
    if q.shape[-1] != HEAD_DIM or keys.shape[-1] != HEAD_DIM or values.shape[-1] != HEAD_DIM:
        return False
    hq, hkv = q.shape[1], keys.shape[1]
    return hq % hkv == 0 and hq // hkv <= MAX_GROUP and values.shape[1] == hkv


def _rows(t: torch.Tensor):
    if t.stride(2) != 1 or t.stride(1) != t.shape[2] or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t, t.stride(0)


def _stream(t):
    return _c.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _p(t):
    return _c.c_void_p(t.data_ptr() if t is not None else 0)


def selected_attention_backward_reference(q, keys, values, sel, out, lse, dout, scale, chunk_rows: int = 256):
    """fp32 statement of the backward pass given the forward's ``out`` and ``lse [Hq, n]``.  ``out`` / ``lse`` may be
    the results of a LARGER softmax (partials merged over shards): probabilities are then ``exp(s - lse)`` of that
    softmax and the gradients are this key set's exact share.  Returns ``(dq, dk, dv)`` in fp32."""
    n, hq, d = q.shape
    hkv = keys.shape[1]
    g = hq // hkv
    dq = torch.zeros(n, hq, d, dtype=torch.float32, device=q.device)
    dk = torch.zeros(keys.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(values.shape, dtype=torch.float32, device=q.device)
    for lo in range(0, n, chunk_rows):
        sl = slice(lo, min(lo + chunk_rows, n))
        s_idx = sel[sl].long()
        ok = (s_idx >= 0) & (s_idx < keys.shape[0])
        safe = s_idx.clamp(0, max(keys.shape[0] - 1, 0))
        kk = keys[safe].float().repeat_interleave(g, 2)                  # [c, L, Hq, d]
        vv = values[safe].float().repeat_interleave(g, 2)
        qf, do = q[sl].float(), dout[sl].float()
        sc = torch.einsum("nhd,nlhd->nhl", qf, kk) * scale
        l = lse[:, sl].t().float()
        has = torch.isfinite(l)
        p = torch.exp(sc - torch.where(has, l, torch.zeros_like(l))[..., None])
        p = torch.where(ok[:, None] & has[..., None], p, torch.zeros_like(p))
        delta = (out[sl].float() * do).sum(-1)                           # [c, Hq]
        dp = torch.einsum("nhd,nlhd->nhl", do, vv)
        ds = p * (dp - delta[..., None]) * scale
        dq[sl] = torch.einsum("nhl,nlhd->nhd", ds, kk)
        c, L = s_idx.shape
        dk_rows = torch.einsum("nhl,nhd->nlhd", ds, qf).reshape(c, L, hkv, g, d).sum(3)
        dv_rows = torch.einsum("nhl,nhd->nlhd", p, do).reshape(c, L, hkv, g, d).sum(3)
        flat = safe.reshape(-1)
        keep = ok.reshape(-1, 1, 1).float()
        dk.index_add_(0, flat, dk_rows.reshape(c * L, hkv, d) * keep)
        dv.index_add_(0, flat, dv_rows.reshape(c * L, hkv, d) * keep)
    return dq, dk, dv


@torch.no_grad()
def selected_attention_forward(q, keys, values, sel, scale) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(out, lse)`` without autograd: the kernel on a GPU (bf16, head dim 128), the fp32 statement elsewhere."""
    if not _kernel_ok(q, keys, values):
        return selected_attention_reference(q, keys, values, sel, scale)
    from aspec_b200 import _native
    from aspec_b200.ops.gemm import status_word
    n, hq, d = q.shape
    q = q.contiguous()
    k, k_ld = _rows(keys)
    v, v_ld = _rows(values)
    sel = sel.to(torch.int32).contiguous()
    out = torch.empty_like(q)
    lse = torch.empty(hq, n, dtype=torch.float32, device=q.device)
    st = status_word(q.device)
    rc = _native.kernels().ab_sel_attn_fwd(_p(q), _p(k), _p(v), _p(sel), _p(out), _p(lse), n, k.shape[0], sel.shape[1], hq,
                                           k.shape[1], d, _c.c_longlong(k_ld), _c.c_longlong(v_ld), _c.c_float(scale),
                                           _p(st), _stream(q))
    if rc != 0:
        raise RuntimeError(f"ab_sel_attn_fwd refused the launch (code {rc})")
    return out, lse


@torch.no_grad()
def selected_attention_backward(q, keys, values, sel, out, lse, dout, scale):
    """``(dq [n, Hq, d] in q's dtype, dk, dv fp32)`` from the forward's ``out`` / ``lse`` (or merged global ones)."""
    if not _kernel_ok(q, keys, values):
        dq, dk, dv = selected_attention_backward_reference(q, keys, values, sel, out, lse, dout, scale)
        return dq.to(q.dtype), dk, dv
    from aspec_b200 import _native
    from aspec_b200.ops.gemm import status_word
    n, hq, d = q.shape
    q = q.contiguous()
    k, k_ld = _rows(keys)
    v, v_ld = _rows(values)
    sel = sel.to(torch.int32).contiguous()
    out, lse, dout = out.contiguous(), lse.float().contiguous(), dout.contiguous()   # named: alive until after the launch
    dq = torch.empty_like(q)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    st = status_word(q.device)
    rc = _native.kernels().ab_sel_attn_bwd(_p(q), _p(k), _p(v), _p(sel), _p(out), _p(lse), _p(dout), _p(dq), _p(dk), _p(dv), n,
                                           k.shape[0], sel.shape[1], hq, k.shape[1], d, _c.c_longlong(k_ld),
                                           _c.c_longlong(v_ld), _c.c_float(scale), _p(st), _stream(q))
    if rc != 0:
        raise RuntimeError(f"ab_sel_attn_bwd refused the launch (code {rc})")
    return dq, dk, dv


class _SelectedAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, keys, values, sel, scale):
        out, lse = selected_attention_forward(q, keys, values, sel, scale)
        ctx.save_for_backward(q, keys, values, sel, out, lse)
        ctx.scale = scale
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, keys, values, sel, out, lse = ctx.saved_tensors
        dq, dk, dv = selected_attention_backward(q, keys, values, sel, out, lse, dout, ctx.scale)
        return dq, dk.to(keys.dtype), dv.to(values.dtype), None, None


def selected_attention(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, sel: torch.Tensor,
                       scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``out [n, Hq, d]`` and ``lse [Hq, n]``: query ``i`` attends the key rows ``sel[i]`` (negative = none).

    Rows whose list is empty give zero output and ``lse = -inf``.  bf16 CUDA tensors with head dim 128 and a group
    size of at most 16 run the tcgen05 kernels; everything else runs the fp32 statement."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    if _kernel_ok(q, keys, values):
        note("sparse_attention", "tcgen05_selected_keys")
        return _SelectedAttentionFn.apply(q.contiguous(), keys, values, sel.to(torch.int32).contiguous(), scale)
    note("sparse_attention", "reference_fp32" + ("_cpu" if not q.is_cuda else ""))
    return selected_attention_reference(q, keys, values, sel, scale)


def indexer_kernel_ok(qi: torch.Tensor, ki: torch.Tensor) -> bool:
    return (qi.is_cuda and qi.dtype == ki.dtype == torch.bfloat16 and qi.shape[1] in (8, 16, 32, 64, 128)
            and qi.shape[2] in (64, 128) and ki.shape[1] == qi.shape[2])


@torch.no_grad()
def indexer_scores(qi: torch.Tensor, ki: torch.Tensor, w: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor,
                   epilogue_groups: int = 0) -> torch.Tensor:
    """``[n, T]`` fp32 scores, ``-inf`` outside ``[lo, hi)``.  ``qi [n, H, d]``, ``ki [T, d]``, ``w [n, H]``.
    ``epilogue_groups`` (1 or 2) forces how many warpgroups drain an accumulator; 0 takes the kernel's default."""
    n, H, d = qi.shape
    T = ki.shape[0]
    if not indexer_kernel_ok(qi, ki):
        note("indexer", "reference_fp32" + ("_cpu" if not qi.is_cuda else ""))
        return indexer_scores_reference(qi, ki, w, lo.long(), hi.long())
    from aspec_b200 import _native
    from aspec_b200.ops.gemm import status_word
    note("indexer", "tcgen05_relu_weighted_head_sum")
    qi = qi.contiguous()
    if ki.stride(1) != 1 or ki.stride(0) % 8 or ki.data_ptr() % 16:
        ki = ki.contiguous()
    out = torch.full((n, T), float("-inf"), dtype=torch.float32, device=qi.device)
    st = status_word(qi.device)
    # converted copies are held in names until after the launch: a temporary freed between two conversions would hand
    # the same block to the next one
    w32, lo32, hi32 = w.float().contiguous(), lo.to(torch.int32).contiguous(), hi.to(torch.int32).contiguous()
    rc = _native.kernels().ab_indexer_scores(_p(qi), _p(ki), _p(w32), _p(lo32), _p(hi32), _p(out),
                                             _c.c_longlong(out.stride(0)), n, T, H, d, _c.c_longlong(ki.stride(0)),
                                             int(epilogue_groups), _p(st), _stream(qi))
    if rc != 0:
        raise RuntimeError(f"ab_indexer_scores refused the launch (code {rc})")
    return out


@torch.no_grad()
def topk_select(scores: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, k: int) -> torch.Tensor:
    """``[n, k]`` int32: ascending indices of the ``k`` largest scores inside ``[lo, hi)`` of each row; ``-1`` pads."""
    if not (scores.is_cuda and scores.dtype == torch.float32 and scores.stride(1) == 1):
        note("topk", "torch")
        return topk_select_reference(scores, lo.long(), hi.long(), k)
    from aspec_b200 import _native
    note("topk", "radix_select")
    n, T = scores.shape
    out = torch.empty(n, k, dtype=torch.int32, device=scores.device)
    lo32, hi32 = lo.to(torch.int32).contiguous(), hi.to(torch.int32).contiguous()
    rc = _native.kernels().ab_topk_select(_p(scores), _c.c_longlong(scores.stride(0)), _p(lo32), _p(hi32), n, T, k, _p(out),
                                          _stream(scores))
    if rc != 0:
        raise RuntimeError(f"ab_topk_select refused the launch (code {rc})")
    return out
