"""ctypes bindings of the interval flash-attention kernels (``csrc/attention_*_sm100.cu``)."""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch

from aspec_b200 import _native
from aspec_b200.ops.gemm import status_word

HEAD_DIM = 128
QK_HEAD_DIMS = (128, 192)          # 192 = materialised-MLA heads (128 "nope" + 64 rotary dims)


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """The tcgen05 kernels cover bf16, value head dim 128, query/key head dim 128 or 192, and group size Hq/Hkv in
    {1,2,4,8,16}."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        return False
    if q.shape[-1] not in QK_HEAD_DIMS or k.shape[-1] != q.shape[-1] or v.shape[-1] != HEAD_DIM:
        return False
    hq, hkv = q.shape[1], k.shape[1]
    return hq % hkv == 0 and (hq // hkv) in (1, 2, 4, 8, 16)


# A dense fp32 score matrix of this many elements (heads x queries x keys) is the most the fallback will allocate.
DENSE_FALLBACK_MAX_SCORES = 1 << 28


def unsupported_shape_fallback(q, k, v, intervals, scale):
    """Shapes outside the kernels' coverage (odd head dims of small auxiliary configurations) run the dense-mask
    statement in fp32 on the device.  It materialises ``heads x queries x keys`` scores, so it refuses problems above
    ``DENSE_FALLBACK_MAX_SCORES`` elements instead of trying to allocate them."""
    from aspec_b200.ops.attention import interval_attention_reference
    scores = q.shape[0] * q.shape[1] * k.shape[0]
    if scores > DENSE_FALLBACK_MAX_SCORES:
        raise ValueError(
            f"attention with head dims ({q.shape[-1]}, {v.shape[-1]}) has no kernel and its dense fallback would need "
            f"{scores} fp32 scores (limit {DENSE_FALLBACK_MAX_SCORES}); supported: bf16, value dim 128, query/key dim 128 or 192")
    return interval_attention_reference(q, k, v, intervals, scale)


def _rows_view(t: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """``[N, H, d]`` with unit strides inside a row (head stride d); returns (tensor, row stride)."""
    if t.stride(2) != 1 or t.stride(1) != t.shape[2] or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t, t.stride(0)


def positions_per_tile(hq: int, hkv: int) -> Optional[int]:
    """Query positions that share one 128-row tile of the kernels (the head group of a key / value head is folded into
    the tile's rows); ``None`` for a group the kernels do not tile in one piece."""
    group = hq // max(hkv, 1)
    return 128 // group if hq % max(hkv, 1) == 0 and group in (1, 2, 4, 8, 16) else None


def forward(q, k, v, intervals, scale, out=None, lse=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q`` may be another GPU's memory mapped here (TMA loads it over NVLink) and ``out`` / ``lse`` may be slots
    in the query owner's memory: that is how context-parallel partial attention moves its data."""
    Q, hq, d = q.shape
    tk, hkv = k.shape[0], k.shape[1]
    q = q.contiguous()
    k, k_ld = _rows_view(k)
    v, v_ld = _rows_view(v)
    out = torch.empty(Q, hq, HEAD_DIM, dtype=q.dtype, device=q.device) if out is None else out
    lse = torch.empty(hq, Q, dtype=torch.float32, device=q.device) if lse is None else lse
    if not (out.is_contiguous() and lse.is_contiguous() and out.shape == (Q, hq, HEAD_DIM) and lse.shape == (hq, Q)):
        raise ValueError("out / lse destinations must be contiguous [Q, H, 128] / [H, Q]")
    st = status_word(q.device)
    rc = _native.kernels().ab_attn_fwd(
        _c.c_void_p(q.data_ptr()), _c.c_void_p(k.data_ptr()), _c.c_void_p(v.data_ptr()),
        _c.c_void_p(intervals.data_ptr()), _c.c_void_p(out.data_ptr()), _c.c_void_p(lse.data_ptr()),
        Q, tk, hq, hkv, d, _c.c_longlong(k_ld), _c.c_longlong(v_ld), _c.c_float(scale),
        _c.c_void_p(st.data_ptr()), _c.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"ab_attn_fwd refused the launch (code {rc})")
    return out, lse


def backward(q, k, v, intervals, out, lse, dout, scale, dq=None):
    Q, hq, d = q.shape
    tk, hkv = k.shape[0], k.shape[1]
    lib = _native.kernels()
    k, k_ld = _rows_view(k)
    v, v_ld = _rows_view(v)
    dq = torch.empty_like(q) if dq is None else dq
    if not (dq.is_contiguous() and dq.shape == q.shape):
        raise ValueError("dq destination must be contiguous [Q, H, d]")
    dk = torch.empty(tk, hkv, d, dtype=q.dtype, device=q.device)
    dv = torch.empty(tk, hkv, HEAD_DIM, dtype=q.dtype, device=q.device)
    delta = torch.empty(hq, Q, dtype=torch.float32, device=q.device)
    pm = 128 // (hq // hkv)
    ranges = torch.empty((Q + pm - 1) // pm, 4, dtype=torch.int32, device=q.device)
    st = status_word(q.device)
    rc = lib.ab_attn_bwd(
        _c.c_void_p(q.data_ptr()), _c.c_void_p(k.data_ptr()), _c.c_void_p(v.data_ptr()),
        _c.c_void_p(intervals.data_ptr()), _c.c_void_p(out.data_ptr()), _c.c_void_p(lse.data_ptr()),
        _c.c_void_p(dout.data_ptr()), _c.c_void_p(delta.data_ptr()), _c.c_void_p(ranges.data_ptr()),
        _c.c_void_p(dq.data_ptr()),
        _c.c_void_p(dk.data_ptr()), _c.c_void_p(dv.data_ptr()), Q, tk, hq, hkv, d,
        _c.c_longlong(k_ld), _c.c_longlong(v_ld), _c.c_float(scale), _c.c_void_p(st.data_ptr()),
        _c.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"ab_attn_bwd refused the launch (code {rc})")
    return dq, dk, dv
