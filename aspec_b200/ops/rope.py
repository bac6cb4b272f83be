"""Rotary position embedding with per-head RMSNorm ("QK-norm + RoPE").

``qk_norm_rope(x, norm_weight, positions, inv_freq, eps)``: for ``x [N, H, d]`` apply RMSNorm over
``d`` with ``norm_weight [d]`` (skipped when ``None``), then rotate-half RoPE at ``positions [N]``.
The CUDA path is one fused kernel for forward and one for backward; the reference implements the
same fusion in CuTe DSL (aspec/kernels/cutedsl/dspark_qk_norm_rope.py:94-424 and ``_bwd.py``).
"""
from __future__ import annotations

from typing import Optional

import torch


class RopeFrequencies:
    """Inverse frequencies kept in fp32 whatever dtype the owning module is cast to (a registered buffer
    would be rounded to bf16 by ``module.to(torch.bfloat16)`` and shift every rotation angle)."""

    def __init__(self, inv_freq):
        self.values = [float(v) for v in inv_freq]
        self._cache = {}

    def get(self, device) -> torch.Tensor:
        key = str(device)
        t = self._cache.get(key)
        if t is None:
            t = torch.tensor(self.values, dtype=torch.float32, device=device)
            self._cache[key] = t
        return t


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, scaling: float = 1.0, axes: Optional[torch.Tensor] = None):
    """``cos, sin [N, d/2]``.  ``positions`` is ``[N]``, or ``[3, N]`` (temporal, height, width) with ``axes [d/2]``
    naming the stream that rotates each frequency (multi-axis RoPE)."""
    if positions.dim() == 2:
        if axes is None:
            raise ValueError("three position streams need the frequency-to-stream table")
        per_freq = positions.float().t()[:, axes.long()]                     # [N, d/2]
        ang = per_freq * inv_freq.float()[None]
    else:
        ang = positions.float()[:, None] * inv_freq.float()[None]
    return torch.cos(ang) * scaling, torch.sin(ang) * scaling


def qk_norm_rope_reference(x: torch.Tensor, norm_weight: Optional[torch.Tensor], positions: torch.Tensor,
                           inv_freq: torch.Tensor, eps: float, scaling: float = 1.0,
                           rope_dim: Optional[int] = None, axes: Optional[torch.Tensor] = None) -> torch.Tensor:
    xf = x.float()
    if norm_weight is not None:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()
    d = x.shape[-1] if rope_dim is None else rope_dim
    cos, sin = rope_tables(positions, inv_freq, scaling, axes)      # [N, d/2]
    cos, sin = cos[:, None], sin[:, None]
    x1, x2 = xf[..., : d // 2], xf[..., d // 2: d]
    rot = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)
    if d < x.shape[-1]:
        rot = torch.cat([rot, xf[..., d:]], -1)
    return rot.to(x.dtype)


class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, norm_weight, positions, inv_freq, eps, scaling, holder):
        from aspec_b200.ops import elementwise_sm100 as E
        y, rstd = E.qk_norm_rope_fwd(x, norm_weight, positions, inv_freq, eps, scaling)
        ctx.save_for_backward(x, norm_weight, positions, inv_freq, rstd)
        ctx.scaling, ctx.holder = scaling, holder
        return y

    @staticmethod
    def backward(ctx, dy):
        from aspec_b200.ops import elementwise_sm100 as E
        x, norm_weight, positions, inv_freq, rstd = ctx.saved_tensors
        dx, dw = E.qk_norm_rope_bwd(dy.contiguous(), x, norm_weight, positions, inv_freq, rstd, ctx.scaling)
        holder = ctx.holder
        main = getattr(holder, "main_grad", None) if holder is not None else None
        if dw is not None and main is not None:
            main.add_(dw)
            holder.main_grad_touched = True
            dw = None
        elif dw is not None:
            dw = dw.to(norm_weight.dtype)
        return dx, dw, None, None, None, None, None


def qk_norm_rope(x: torch.Tensor, norm_weight: Optional[torch.Tensor], positions: torch.Tensor,
                 inv_freq: torch.Tensor, eps: float, scaling: float = 1.0, axes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [N, H, d]`` -> normalised + rotated, same shape and dtype.

    ``positions [3, N]`` with ``axes`` is multi-axis RoPE.  Rows whose three streams agree (all text) are exactly
    ordinary RoPE and take the fused kernel; rows with distinct streams use the fp32 statement."""
    if positions.dim() == 2:
        if bool((positions[0] == positions[1]).all() & (positions[0] == positions[2]).all()):
            positions = positions[0]
        else:
            return qk_norm_rope_reference(x, norm_weight, positions, inv_freq, eps, scaling, axes=axes)
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] in (64, 128, 256) and x.numel():
        holder = norm_weight if isinstance(norm_weight, torch.nn.Parameter) else None
        return _QKNormRopeFn.apply(x.contiguous(), norm_weight, positions.contiguous().to(torch.int32),
                                   inv_freq.float().contiguous(), eps, scaling, holder)
    return qk_norm_rope_reference(x, norm_weight, positions, inv_freq, eps, scaling)
