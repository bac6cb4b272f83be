"""SwiGLU on a fused ``[gate | up]`` projection (kernel on CUDA, reference on CPU).

``swiglu(gu)`` with ``gu [..., 2I]`` returns ``silu(gu[..., :I]) * gu[..., I:]``; ``clamp > 0`` applies the
Ling-MoE limits ``gate <= clamp`` and ``|up| <= clamp`` first (aspec/models/draft/ling_moe.py:34-44).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def swiglu_reference(gu: torch.Tensor, clamp: float = 0.0) -> torch.Tensor:
    g, u = gu.float().chunk(2, dim=-1)
    if clamp > 0:
        g = g.clamp(max=clamp)
        u = u.clamp(min=-clamp, max=clamp)
    return (F.silu(g) * u).to(gu.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, clamp):
        from aspec_b200.ops import elementwise_sm100 as E
        ctx.save_for_backward(gu)
        ctx.clamp = clamp
        return E.swiglu_fwd(gu, clamp)

    @staticmethod
    def backward(ctx, dact):
        from aspec_b200.ops import elementwise_sm100 as E
        (gu,) = ctx.saved_tensors
        return E.swiglu_bwd(gu, dact.contiguous(), ctx.clamp), None


def swiglu(gu: torch.Tensor, clamp: float = 0.0) -> torch.Tensor:
    if gu.is_cuda and gu.dtype == torch.bfloat16 and gu.shape[-1] % 16 == 0 and gu.numel():
        lead = gu.shape[:-1]
        out = _SwiGLUFn.apply(gu.reshape(-1, gu.shape[-1]).contiguous(), float(clamp))
        return out.view(*lead, gu.shape[-1] // 2)
    return swiglu_reference(gu, clamp)


def swiglu_backward(gu: torch.Tensor, dact: torch.Tensor, clamp: float = 0.0) -> torch.Tensor:
    """``d gu [..., 2I]`` from ``d act [..., I]`` (explicit backward for code that manages its own graph)."""
    if gu.is_cuda and gu.dtype == torch.bfloat16 and gu.shape[-1] % 16 == 0 and gu.numel():
        from aspec_b200.ops import elementwise_sm100 as E
        return E.swiglu_bwd(gu.reshape(-1, gu.shape[-1]).contiguous(), dact.reshape(-1, dact.shape[-1]).contiguous(), float(clamp)).view(gu.shape)
    if gu.numel() == 0:
        return torch.zeros_like(gu)
    with torch.enable_grad():            # callers sit inside an autograd backward, where recording is off
        g = gu.detach().clone().requires_grad_(True)
        swiglu_reference(g, clamp).backward(dact.to(gu.dtype))
    return g.grad
