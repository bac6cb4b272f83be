"""Grouped bf16 GEMM (``csrc/grouped_gemm_sm100.cu``): many small problems, one persistent tcgen05 launch.

Two shapes of problem list cover a mixture-of-experts layer:

* ``rows_gemm`` - every problem multiplies a run of token rows (taken from one of several row buffers, which may be
  views of other GPUs' memory) with one matrix of a stacked weight tensor and stores the rows into one of several
  output buffers: expert forward, input gradients;
* ``wgrad_gemm`` - every problem reduces over token rows, possibly drawn from several buffers: expert weight
  gradients.  One of the two operands of each run must be zero-padded to a multiple of 64 rows (``padded_offsets``)
  and the other finite, because the last 64-row block of a run reads past its end.

The reference loops over experts in Python with one library GEMM each (aspec/models/draft/ling_moe.py:101-115).
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import numpy as np
import torch

from aspec_b200 import _native
from aspec_b200.ops.gemm import status_word

BM, BN, BK = 128, 256, 64
MAX_MAPS = 12

_TILE = np.dtype([("d", "<u8"), ("ldd", "<i8"), ("rows", "<i4"), ("cols", "<i4"), ("seg0", "<i4"), ("nseg", "<i4")])
_SEG = np.dtype([("a_map", "<i4"), ("a_mn", "<i4"), ("a_k", "<i4"), ("b_map", "<i4"), ("b_mn", "<i4"), ("b_k", "<i4"),
                 ("k_blocks", "<i4"), ("pad", "<i4")])
assert _TILE.itemsize == 32 and _SEG.itemsize == 32


class _GroupedOperand(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("rows", ctypes.c_longlong), ("cols", ctypes.c_longlong),
                ("ld", ctypes.c_longlong), ("role", ctypes.c_int), ("mn_major", ctypes.c_int)]


def padded_offsets(counts: Sequence[int], multiple: int = BK):
    """Start row of every run when each run is padded to ``multiple`` rows; returns ``(offsets, total)``."""
    c = np.asarray(counts, dtype=np.int64)
    padded = -(-c // multiple) * multiple
    off = np.concatenate([[0], np.cumsum(padded)])
    return off[:-1], int(off[-1])


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.bfloat16 or t.stride(-1) != 1:
        raise ValueError("grouped GEMM operands must be bf16 with unit inner stride")
    return t.reshape(-1, t.shape[-1]) if t.dim() == 3 else t


def _launch(operands, tiles: np.ndarray, segs: np.ndarray, a_mn: bool, b_mn: bool, fp32: bool, alpha: float, device,
            max_ctas: int = 0) -> None:
    if len(operands) > MAX_MAPS:
        raise ValueError(f"at most {MAX_MAPS} operand buffers per grouped launch")
    if len(tiles) == 0:
        return
    ops = (_GroupedOperand * len(operands))()
    for i, (t, role) in enumerate(operands):
        ops[i] = _GroupedOperand(t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), role, int(a_mn if role == 0 else b_mn))
    table = np.concatenate([tiles.view(np.uint8), segs.view(np.uint8)])
    dev = torch.from_numpy(table).to(device, non_blocking=True)
    seg_ptr = dev.data_ptr() + tiles.nbytes
    rc = _native.kernels().ab_grouped_gemm_bf16(
        ctypes.c_int(len(operands)), ops, ctypes.c_void_p(dev.data_ptr()), ctypes.c_int(len(tiles)),
        ctypes.c_void_p(seg_ptr), ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)), ctypes.c_int(int(fp32)),
        ctypes.c_float(alpha), ctypes.c_void_p(status_word(device).data_ptr()), ctypes.c_int(max_ctas),
        ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"ab_grouped_gemm_bf16 refused the launch (code {rc})")


NATIVE_PLANNER = True          # tables from the C++ runtime (csrc/runtime/grouped_plan.cpp); False: the array-library statement


def _i64(v) -> np.ndarray:
    return np.ascontiguousarray(v, dtype=np.int64)


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def _plan_rows_native(src, a_row, rows, expert, dst, out_row, base, ldd, esize, N, K, b_map, b_t):
    lib = _native.runtime()
    lib.ab_plan_rows_count.restype = ctypes.c_int64
    lib.ab_plan_rows_gemm.restype = ctypes.c_int64
    src, a_row, rows, expert, dst, out_row, ldd = (_i64(v) for v in (src, a_row, rows, expert, dst, out_row, ldd))
    base = np.ascontiguousarray(base, dtype=np.uint64)
    total = int(lib.ab_plan_rows_count(ctypes.c_int(len(rows)), _ptr(rows), ctypes.c_int64(N)))
    tiles, segs = np.empty(total, dtype=_TILE), np.empty(total, dtype=_SEG)
    lib.ab_plan_rows_gemm(ctypes.c_int(len(rows)), _ptr(src), _ptr(a_row), _ptr(rows), _ptr(expert), _ptr(dst), _ptr(out_row),
                          _ptr(base), _ptr(ldd), ctypes.c_int(esize), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(b_map),
                          ctypes.c_int(int(b_t)), _ptr(tiles), _ptr(segs))
    return tiles, segs


def _plan_rows_numpy(src, a_row, rows, expert, dst, out_row, base, ldd, esize, N, K, b_map, b_t):
    m_tiles = -(-rows // BM)
    n_tiles = -(-N // BN)
    per = m_tiles * n_tiles
    total = int(per.sum())
    prob = np.repeat(np.arange(len(rows)), per)
    within = np.arange(total) - np.repeat(np.cumsum(per) - per, per)
    nt = within // m_tiles[prob]                      # n-tile major inside a problem: CTAs in flight share B
    mt = within - nt * m_tiles[prob]
    tiles = np.zeros(total, dtype=_TILE)
    row0 = out_row[prob] + mt * BM
    tiles["d"] = base[dst[prob]] + ((row0 * ldd[dst[prob]] + nt * BN) * esize).astype(np.uint64)
    tiles["ldd"] = ldd[dst[prob]]
    tiles["rows"] = np.minimum(BM, rows[prob] - mt * BM)
    tiles["cols"] = np.minimum(BN, N - nt * BN)
    tiles["seg0"] = np.arange(total)
    tiles["nseg"] = 1
    segs = np.zeros(total, dtype=_SEG)
    segs["a_map"] = src[prob]
    segs["a_mn"] = a_row[prob] + mt * BM
    segs["a_k"] = 0
    segs["b_map"] = b_map
    if b_t:
        segs["b_mn"] = nt * BN
        segs["b_k"] = expert[prob] * K
    else:
        segs["b_mn"] = expert[prob] * N + nt * BN
        segs["b_k"] = 0
    segs["k_blocks"] = -(-K // BK)
    return tiles, segs


def _plan_wgrad_native(expert, a_src, a_row, b_src, b_row, rows, E, Ma, Nb, out, esize, b_map0):
    lib = _native.runtime()
    lib.ab_plan_wgrad_gemm.restype = ctypes.c_int64
    expert, a_src, a_row, b_src, b_row, rows = (_i64(v) for v in (expert, a_src, a_row, b_src, b_row, rows))
    per = -(-Ma // BM) * -(-Nb // BN)
    n_seg = len(rows) * per
    tiles, segs = np.empty(E * per, dtype=_TILE), np.empty(n_seg, dtype=_SEG)
    lib.ab_plan_wgrad_gemm(ctypes.c_int(len(rows)), _ptr(expert), _ptr(a_src), _ptr(a_row), _ptr(b_src), _ptr(b_row), _ptr(rows),
                           ctypes.c_int(E), ctypes.c_int64(Ma), ctypes.c_int64(Nb), ctypes.c_uint64(out.data_ptr()),
                           ctypes.c_int64(out.stride(0)), ctypes.c_int64(out.stride(1)), ctypes.c_int(esize), ctypes.c_int(b_map0),
                           _ptr(tiles), _ptr(segs))
    return tiles, segs


def rows_gemm(a_bufs: List[torch.Tensor], weights: torch.Tensor, out_bufs: List[torch.Tensor], *, src, a_row, rows,
              expert, dst, out_row, b_t: bool = False, alpha: float = 1.0) -> None:
    """For every problem ``i``: ``out_bufs[dst[i]][out_row[i] : out_row[i] + rows[i]] = a_bufs[src[i]][a_row[i] : ...] @ W_i``.

    ``weights`` is the stacked tensor: ``[E, N, K]`` (``b_t=False``, ``W_i = weights[expert[i]].T``) or ``[E, K, N]``
    (``b_t=True``, ``W_i = weights[expert[i]]``).  All index arguments are host sequences of equal length.
    """
    src, a_row, rows, expert, dst, out_row = (np.asarray(v, dtype=np.int64) for v in (src, a_row, rows, expert, dst, out_row))
    keep = rows > 0
    src, a_row, rows, expert, dst, out_row = (v[keep] for v in (src, a_row, rows, expert, dst, out_row))
    if len(rows) == 0:
        return
    E = weights.shape[0]
    if b_t:
        K, N = weights.shape[1], weights.shape[2]
    else:
        N, K = weights.shape[1], weights.shape[2]
    a_bufs = [_as_2d(a) for a in a_bufs]
    for a in a_bufs:
        if a.shape[1] != K:
            raise ValueError("row buffers must have the reduction extent as their width")
    w2d = _as_2d(weights)
    operands = [(a, 0) for a in a_bufs] + [(w2d, 1)]
    b_map = len(a_bufs)
    out_dtype = out_bufs[0].dtype
    esize = 4 if out_dtype == torch.float32 else 2
    for o in out_bufs:
        if o.dtype != out_dtype or o.stride(1) != 1 or o.shape[1] < N:
            raise ValueError("output buffers must share a dtype, have unit inner stride and at least N columns")
    base = np.array([o.data_ptr() for o in out_bufs], dtype=np.uint64)
    ldd = np.array([o.stride(0) for o in out_bufs], dtype=np.int64)
    plan = _plan_rows_native if NATIVE_PLANNER else _plan_rows_numpy
    tiles, segs = plan(src, a_row, rows, expert, dst, out_row, base, ldd, esize, N, K, b_map, b_t)
    if b_t and K % BK and E > 1:
        raise ValueError("a transposed stacked weight needs its reduction extent to be a multiple of 64")
    _launch(operands, tiles, segs, False, b_t, out_dtype == torch.float32, alpha, a_bufs[0].device)


def _plan_wgrad_numpy(expert, a_src, a_row, b_src, b_row, rows, E, Ma, Nb, out, esize, b_map0):
    runs_per_expert = np.bincount(expert, minlength=E)
    run0 = np.cumsum(runs_per_expert) - runs_per_expert
    m_tiles, n_tiles = -(-Ma // BM), -(-Nb // BN)
    per = m_tiles * n_tiles
    total = E * per
    e_of = np.repeat(np.arange(E), per)
    within = np.arange(total) - e_of * per
    nt = within // m_tiles
    mt = within - nt * m_tiles
    tiles = np.zeros(total, dtype=_TILE)
    tiles["d"] = np.uint64(out.data_ptr()) + ((e_of * out.stride(0) + mt * BM * out.stride(1) + nt * BN) * esize).astype(np.uint64)
    tiles["ldd"] = out.stride(1)
    tiles["rows"] = np.minimum(BM, Ma - mt * BM)
    tiles["cols"] = np.minimum(BN, Nb - nt * BN)
    nseg = runs_per_expert[e_of]
    tiles["nseg"] = nseg
    seg_start = np.cumsum(nseg) - nseg
    tiles["seg0"] = seg_start
    n_seg_total = int(nseg.sum())
    tile_of = np.repeat(np.arange(total), nseg)
    run = run0[e_of[tile_of]] + (np.arange(n_seg_total) - seg_start[tile_of])
    segs = np.zeros(n_seg_total, dtype=_SEG)
    segs["a_map"] = a_src[run]
    segs["a_mn"] = mt[tile_of] * BM
    segs["a_k"] = a_row[run]
    segs["b_map"] = b_map0 + b_src[run]
    segs["b_mn"] = nt[tile_of] * BN
    segs["b_k"] = b_row[run]
    segs["k_blocks"] = -(-rows[run] // BK)
    return tiles, segs


def wgrad_gemm(a_bufs: List[torch.Tensor], b_bufs: List[torch.Tensor], out: torch.Tensor, *, expert, a_src, a_row, b_src,
               b_row, rows, alpha: float = 1.0) -> None:
    """``out[e] = sum over runs i with expert[i] == e of  A_i^T @ B_i`` with ``A_i = a_bufs[a_src[i]][a_row[i] : + rows[i]]``
    (``[rows, Ma]``) and ``B_i`` likewise (``[rows, Nb]``); ``out`` is ``[E, Ma, Nb]`` fp32 or bf16 and is fully written
    (experts without rows get zeros)."""
    expert, a_src, a_row, b_src, b_row, rows = (np.asarray(v, dtype=np.int64) for v in (expert, a_src, a_row, b_src, b_row, rows))
    E, Ma, Nb = out.shape
    keep = rows > 0
    expert, a_src, a_row, b_src, b_row, rows = (v[keep] for v in (expert, a_src, a_row, b_src, b_row, rows))
    order = np.argsort(expert, kind="stable")
    expert, a_src, a_row, b_src, b_row, rows = (v[order] for v in (expert, a_src, a_row, b_src, b_row, rows))
    a_bufs, b_bufs = [_as_2d(a) for a in a_bufs], [_as_2d(b) for b in b_bufs]
    operands = [(a, 0) for a in a_bufs] + [(b, 1) for b in b_bufs]
    esize = 4 if out.dtype == torch.float32 else 2
    if NATIVE_PLANNER:
        tiles, segs = _plan_wgrad_native(expert, a_src, a_row, b_src, b_row, rows, E, Ma, Nb, out, esize, len(a_bufs))
    else:
        tiles, segs = _plan_wgrad_numpy(expert, a_src, a_row, b_src, b_row, rows, E, Ma, Nb, out, esize, len(a_bufs))
    if out.stride(2) != 1:
        raise ValueError("output must have unit inner stride")
    _launch(operands, tiles, segs, True, True, out.dtype == torch.float32, alpha, out.device)


class _GroupedExperts(torch.autograd.Function):
    """SwiGLU experts over tokens sorted by expert: five grouped launches forward + backward instead of seven GEMMs per expert."""

    @staticmethod
    def forward(ctx, x, gate_up, down, counts, clamp):
        from aspec_b200.ops.activation import swiglu
        counts = np.asarray(counts, dtype=np.int64)
        E, I2, D = gate_up.shape
        start = np.cumsum(counts) - counts
        pstart, ptotal = padded_offsets(counts)
        idx = np.arange(E)
        zeros = np.zeros(E, dtype=np.int64)
        gu = torch.zeros(ptotal, I2, dtype=x.dtype, device=x.device)          # padded layout: zero rows between experts
        rows_gemm([x], gate_up, [gu], src=zeros, a_row=start, rows=counts, expert=idx, dst=zeros, out_row=pstart)
        act = swiglu(gu, clamp)
        y = torch.empty(x.shape[0], D, dtype=x.dtype, device=x.device)
        rows_gemm([act], down, [y], src=zeros, a_row=pstart, rows=counts, expert=idx, dst=zeros, out_row=start)
        ctx.save_for_backward(x, gate_up, down, gu, act)
        ctx.layout = (counts, start, pstart, ptotal, clamp)
        return y

    @staticmethod
    def backward(ctx, dy):
        from aspec_b200.ops.activation import swiglu_backward
        x, gate_up, down, gu, act = ctx.saved_tensors
        counts, start, pstart, ptotal, clamp = ctx.layout
        E, I2, D = gate_up.shape
        idx, zeros = np.arange(E), np.zeros(E, dtype=np.int64)
        dy = dy.contiguous()
        d_act = torch.zeros(ptotal, I2 // 2, dtype=x.dtype, device=x.device)
        rows_gemm([dy], down, [d_act], src=zeros, a_row=start, rows=counts, expert=idx, dst=zeros, out_row=pstart, b_t=True)
        d_gu = swiglu_backward(gu, d_act, clamp)                               # zero rows stay zero
        dx = torch.empty_like(x)
        rows_gemm([d_gu], gate_up, [dx], src=zeros, a_row=pstart, rows=counts, expert=idx, dst=zeros, out_row=start, b_t=True)
        d_down = torch.empty(down.shape, dtype=torch.float32, device=x.device)
        wgrad_gemm([dy], [act], d_down, expert=idx, a_src=zeros, a_row=start, b_src=zeros, b_row=pstart, rows=counts)
        d_gate_up = torch.empty(gate_up.shape, dtype=torch.float32, device=x.device)
        wgrad_gemm([d_gu], [x], d_gate_up, expert=idx, a_src=zeros, a_row=pstart, b_src=zeros, b_row=start, rows=counts)
        return dx, d_gate_up.to(gate_up.dtype), d_down.to(down.dtype), None, None


def grouped_experts(x_sorted: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, counts, clamp: float = 0.0) -> torch.Tensor:
    """``x_sorted [N, D]`` grouped by expert with ``counts[e]`` rows each; ``gate_up [E, 2I, D]``, ``down [E, D, I]``."""
    return _GroupedExperts.apply(x_sorted.contiguous(), gate_up, down, counts, float(clamp))
