"""ctypes bindings of the memory-bound sm_100a kernels (``csrc/elementwise_sm100.cu``)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from aspec_b200 import _native

_c = ctypes


def _p(t: Optional[torch.Tensor]):
    return _c.c_void_p(t.data_ptr() if t is not None else 0)


def _stream(t: torch.Tensor):
    return _c.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _check(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed to launch (code {rc})")


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    rows, H = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(_native.kernels().ab_rmsnorm_fwd(_p(x), _p(w), _p(y), _p(rstd), rows, H, _c.c_float(eps),
                                            _stream(x)), "ab_rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy, x, w, rstd) -> Tuple[torch.Tensor, torch.Tensor]:
    rows, H = x.shape
    dx = torch.empty_like(x)
    dw = torch.zeros(H, dtype=torch.float32, device=x.device)
    _check(_native.kernels().ab_rmsnorm_bwd(_p(dy), _p(x), _p(w), _p(rstd), _p(dx), _p(dw), rows, H,
                                            _stream(x)), "ab_rmsnorm_bwd")
    return dx, dw


def qk_norm_rope_fwd(x, w, pos, inv_freq, eps, scaling):
    N, H, D = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(N * H, dtype=torch.float32, device=x.device)
    _check(_native.kernels().ab_qk_norm_rope_fwd(_p(x), _p(w), _p(pos), _p(inv_freq), _p(y), _p(rstd),
                                                 _c.c_longlong(N), H, D, _c.c_float(eps),
                                                 _c.c_float(scaling), _stream(x)), "ab_qk_norm_rope_fwd")
    return y, rstd


def qk_norm_rope_bwd(dy, x, w, pos, inv_freq, rstd, scaling):
    N, H, D = x.shape
    dx = torch.empty_like(x)
    dw = torch.zeros(D, dtype=torch.float32, device=x.device) if w is not None else None
    _check(_native.kernels().ab_qk_norm_rope_bwd(_p(dy), _p(x), _p(w), _p(pos), _p(inv_freq), _p(rstd),
                                                 _p(dx), _p(dw), _c.c_longlong(N), H, D,
                                                 _c.c_float(scaling), _stream(x)), "ab_qk_norm_rope_bwd")
    return dx, dw


def swiglu_fwd(gu: torch.Tensor, clamp: float = 0.0) -> torch.Tensor:
    R, two_i = gu.shape
    act = torch.empty(R, two_i // 2, dtype=gu.dtype, device=gu.device)
    _check(_native.kernels().ab_swiglu_fwd(_p(gu), _p(act), _c.c_longlong(R), two_i // 2,
                                           _c.c_float(clamp), _stream(gu)), "ab_swiglu_fwd")
    return act


def swiglu_bwd(gu: torch.Tensor, dact: torch.Tensor, clamp: float = 0.0) -> torch.Tensor:
    R, two_i = gu.shape
    dgu = torch.empty_like(gu)
    _check(_native.kernels().ab_swiglu_bwd(_p(gu), _p(dact), _p(dgu), _c.c_longlong(R), two_i // 2,
                                           _c.c_float(clamp), _stream(gu)), "ab_swiglu_bwd")
    return dgu


def merge_rowstats(stats: torch.Tensor) -> torch.Tensor:
    nt, M, _ = stats.shape
    lse = torch.empty(M, dtype=torch.float32, device=stats.device)
    _check(_native.kernels().ab_merge_rowstats(_p(stats), _p(lse), nt, M, _stream(stats)), "ab_merge_rowstats")
    return lse


def vocab_loss(logits, teacher, lse_s, lse_t, t_index, labels, weight, *, mode: int, a_ce: float,
               a_l1: float, write_grad: bool):
    """In place: ``logits`` becomes d(loss)/d(logits) when ``write_grad``.  Returns (ce, l1, correct)."""
    R, V = logits.shape
    dev = logits.device
    ce = torch.empty(R, dtype=torch.float32, device=dev)
    l1 = torch.empty(R, dtype=torch.float32, device=dev)
    correct = torch.empty(R, dtype=torch.float32, device=dev)
    _check(_native.kernels().ab_vocab_loss(
        _p(logits), _p(teacher), _p(lse_s), _p(lse_t), _p(t_index), _p(labels), _p(weight), _p(ce),
        _p(l1), _p(correct), _c.c_longlong(logits.stride(0)),
        _c.c_longlong(teacher.stride(0) if teacher is not None else 0), R, V, mode, _c.c_float(a_ce),
        _c.c_float(a_l1), 1 if write_grad else 0, _stream(logits)), "ab_vocab_loss")
    return ce, l1, correct


def vocab_loss_shard(logits, teacher, lse_s, lse_t, t_index, labels, weight, ce_part, l1_part, c_io, best_val, best_idx, *,
                     vocab_offset: int, a_ce: float, a_l1: float, phase: int) -> None:
    """Vocabulary-sharded loss: ``phase=1`` writes this shard's statistics, ``phase=2`` turns ``logits`` into the
    gradient using the globally summed ``c_io``.  ``lse_s`` / ``lse_t`` are normalisers over the full vocabulary."""
    R, V = logits.shape
    _check(_native.kernels().ab_vocab_loss_shard(
        _p(logits), _p(teacher), _p(lse_s), _p(lse_t), _p(t_index), _p(labels), _p(weight), _p(ce_part), _p(l1_part),
        _p(c_io), _p(best_val), _p(best_idx), _c.c_longlong(logits.stride(0)),
        _c.c_longlong(teacher.stride(0) if teacher is not None else 0), R, V, _c.c_longlong(vocab_offset),
        _c.c_float(a_ce), _c.c_float(a_l1), int(phase), _stream(logits)), "ab_vocab_loss_shard")


def sumsq(g: torch.Tensor, out: torch.Tensor) -> None:
    _check(_native.kernels().ab_sumsq(_p(g), _c.c_longlong(g.numel()), _p(out), _stream(g)), "ab_sumsq")


def adamw(master, grad, m, v, param, ctrl, *, lr, beta1, beta2, eps, wd, step, max_norm) -> None:
    """``step=None``: the kernel takes the bias-correction step from ``ctrl[4]`` (applied updates, kept on the device)."""
    bc1 = 0.0 if step is None else 1.0 - beta1 ** step
    bc2 = 0.0 if step is None else 1.0 - beta2 ** step
    f = _c.c_float
    _check(_native.kernels().ab_adamw(_p(master), _p(grad), _p(m), _p(v), _p(param),
                                      _c.c_longlong(master.numel()), _p(ctrl), f(lr), f(beta1), f(beta2),
                                      f(eps), f(wd), f(bc1), f(bc2), f(max_norm), _stream(master)),
           "ab_adamw")


def scale_bf16_(x: torch.Tensor, scalar: torch.Tensor) -> torch.Tensor:
    _check(_native.kernels().ab_scale_bf16(_p(x), _c.c_longlong(x.numel()), _p(scalar), _stream(x)),
           "ab_scale_bf16")
    return x


def cast_scale(x_fp32: torch.Tensor, scalar: Optional[torch.Tensor] = None, mult: float = 1.0) -> torch.Tensor:
    out = torch.empty(x_fp32.shape, dtype=torch.bfloat16, device=x_fp32.device)
    _check(_native.kernels().ab_cast_scale(_p(x_fp32), _p(out), _c.c_longlong(x_fp32.numel()), _p(scalar),
                                           _c.c_float(mult), _stream(x_fp32)), "ab_cast_scale")
    return out
