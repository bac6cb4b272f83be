"""bf16 GEMM on the tcgen05 tensor cores (``csrc/gemm_sm100.cu``).

``gemm(a, b)`` computes ``a @ b.T`` for bf16 CUDA tensors.  Either operand can be
given "as stored the other way round" (``a_t=True`` means the tensor passed is
``a.T`` in memory, i.e. ``[K, M]``), which maps to the MN-major shared-memory
descriptors of the kernel - no transposed copy is ever made.  The three GEMMs of
a Linear layer therefore are::

    y  = gemm(x, w)                       # [M,K] x [N,K]^T
    dx = gemm(dy, w, b_t=True)            # [M,N] x ([N,K] read as B^T stored)
    dw = gemm(dy, x, a_t=True, b_t=True)  # dy^T x  -> [N,K]

The reference routes all of these through cuBLAS via ``nn.Linear``
(aspec/models/draft/dflash.py:432-507, 968-981).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from aspec_b200 import _native

EPI_STORE, EPI_ROWSTATS, EPI_SWIGLU = 0, 1, 2
TILE_N = 256


NUM_SMS = 148
# CTA-pair (cta_group::2) kernels by default; AB_GEMM_PAIR=0/1 overrides
PAIR_DEFAULT = os.environ.get("AB_GEMM_PAIR", "1") == "1"


def _wave_efficiency(M: int, N: int, pair: bool = False) -> float:
    tiles = -(-M // (256 if pair else 128)) * -(-N // TILE_N)
    waves = tiles / (NUM_SMS // 2 if pair else NUM_SMS)
    return waves / math.ceil(waves)


def _mirror_ptrs(mirrors):
    """``mirrors``: bf16 2-D tensors (possibly views of another GPU's memory) with the output's shape."""
    if not mirrors:
        return None
    return (ctypes.c_void_p * len(mirrors))(*[m.data_ptr() for m in mirrors])


def _mirror_lds(mirrors):
    if not mirrors:
        return None
    return (ctypes.c_longlong * len(mirrors))(*[m.stride(0) for m in mirrors])


class _Operand(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("ld", ctypes.c_longlong), ("mn_major", ctypes.c_int)]


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait ran out."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device) -> None:
    """Raise if any kernel launched so far reported a timeout (synchronises)."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"aspec_b200 kernel reported status {code} (1 = wait timeout)")


def _operand(t: torch.Tensor, transposed: bool) -> _Operand:
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("GEMM operands must be 2-D bf16 with unit inner stride")
    return _Operand(t.data_ptr(), t.stride(0), 1 if transposed else 0)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
         a2: Optional[torch.Tensor] = None, b2: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         addend: Optional[torch.Tensor] = None, alpha: float = 1.0,
         epilogue: int = EPI_STORE, stats: Optional[torch.Tensor] = None,
         logit_scale: float = 1.0, max_ctas: int = 0, stream_k: Optional[bool] = None,
         mirrors=None, scatter_cols: int = 0, cta_pair: Optional[bool] = None) -> torch.Tensor:
    """``alpha * (A @ B^T [+ A2 @ B2^T]) [+ addend]`` with a fused epilogue.

    ``mirrors``: extra bf16 destinations (up to 8, possibly views of other GPUs' memory) that receive every output
    tile straight from the epilogue.  With ``scatter_cols > 0`` the output is scattered instead: columns
    ``[m * scatter_cols, (m + 1) * scatter_cols)`` go only to ``mirrors[m]`` (its own column origin at 0) and no
    local result is written - the sequence-to-head all-to-all of Ulysses attention done by the GEMM's stores.

    ``cta_pair``: run every 256 x 256 output tile on two CTAs of a cluster (``tcgen05`` ``cta_group::2``: each CTA
    stages half of B, one thread issues 256-row MMAs for both).  ``None`` takes the module default ``PAIR_DEFAULT``.

    ``stream_k=None`` picks the schedule: when whole output tiles would leave more than ~12 % of the last
    wave of CTAs idle (for example 448 tiles on 148 SMs), the (tile, k-block) space is divided evenly
    over the CTAs instead and split tiles are combined with fp32 reductions.  A bf16 result then goes
    through an fp32 workspace and one cast pass.
    """
    if cta_pair is None:
        cta_pair = PAIR_DEFAULT
    M = a.shape[1] if a_t else a.shape[0]
    K = a.shape[0] if a_t else a.shape[1]
    N = b.shape[1] if b_t else b.shape[0]
    Kb = b.shape[0] if b_t else b.shape[1]
    if K != Kb:
        raise ValueError(f"reduction extents differ: {K} vs {Kb}")
    K2 = 0
    if a2 is not None:
        K2 = a2.shape[0] if a_t else a2.shape[1]
    n_out = N // 2 if epilogue == EPI_SWIGLU else N
    if mirrors:
        stream_k = False
    inplace_acc = addend is not None and out is not None and addend.data_ptr() == out.data_ptr()
    if stream_k is None:
        tiles = -(-M // (256 if cta_pair else 128)) * -(-N // TILE_N)
        units = NUM_SMS // 2 if cta_pair else NUM_SMS
        stream_k = (epilogue == EPI_STORE and (addend is None or inplace_acc)
                    and ((_wave_efficiency(M, N, cta_pair) < 0.88 and (K + K2) >= 8192)
                         or (tiles < units // 2 and (K + K2) >= 16384)))
    workspace_for = None
    if stream_k:
        if epilogue != EPI_STORE or not (addend is None or inplace_acc):
            raise ValueError("stream-K needs the plain store epilogue without a separate addend")
        want_dtype = out.dtype if out is not None else out_dtype
        if want_dtype != torch.float32:
            workspace_for = out if out is not None else True
            out = torch.zeros((M, N), dtype=torch.float32, device=a.device)
        elif out is None:
            out = torch.zeros((M, N), dtype=torch.float32, device=a.device)
        elif not inplace_acc:
            out.zero_()
    if scatter_cols:
        if not mirrors or scatter_cols % 32 or scatter_cols * len(mirrors) < N or addend is not None:
            raise ValueError("scatter needs mirrors covering all columns in multiples of 32 and no addend")
        out = mirrors[0]                       # placeholder for the descriptor; never written in scatter mode
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=a.device)
    if out.stride(1) != 1:
        raise ValueError("output must have unit inner stride")
    if addend is not None and (addend.dtype != out.dtype or addend.stride() != out.stride()):
        raise ValueError("addend must match the output's dtype and strides")
    lib = _native.kernels()
    oa, ob = _operand(a, a_t), _operand(b, b_t)
    oa2 = _operand(a2, a_t) if a2 is not None else oa
    ob2 = _operand(b2, b_t) if b2 is not None else ob
    st = status_word(a.device)
    rc = lib.ab_gemm_bf16(
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(K2),
        ctypes.byref(oa), ctypes.byref(ob), ctypes.byref(oa2), ctypes.byref(ob2),
        ctypes.c_void_p(out.data_ptr()), ctypes.c_longlong(out.stride(0)),
        ctypes.c_int(1 if out.dtype == torch.float32 else 0),
        ctypes.c_void_p(addend.data_ptr() if addend is not None else 0),
        ctypes.c_float(alpha), ctypes.c_int(epilogue),
        ctypes.c_void_p(stats.data_ptr() if stats is not None else 0),
        ctypes.c_float(logit_scale), ctypes.c_void_p(st.data_ptr()),
        ctypes.c_int(max_ctas), ctypes.c_int(1 if stream_k else 0),
        ctypes.c_int(len(mirrors) if mirrors else 0), _mirror_ptrs(mirrors), _mirror_lds(mirrors),
        ctypes.c_int(int(scatter_cols)), ctypes.c_int(1 if cta_pair else 0),
        ctypes.c_void_p(torch.cuda.current_stream(a.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"ab_gemm_bf16 refused the launch (code {rc}) for M={M} N={N} K={K}")
    if scatter_cols:
        return None
    if workspace_for is not None:
        from aspec_b200.ops import elementwise_sm100 as E
        cast = E.cast_scale(out)
        if workspace_for is True:
            return cast
        workspace_for.copy_(cast)
        return workspace_for
    return out
