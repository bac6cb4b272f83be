"""RMSNorm (fused sm_100a kernel on CUDA, fp32 PyTorch reference on CPU).

``y = x * rsqrt(mean(x^2) + eps) * weight`` with fp32 statistics.  The reference uses Quack's
CuTe-DSL RMSNorm when present (aspec/models/draft/dflash.py:175-188).
"""
from __future__ import annotations

import torch


def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * weight.float()).to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, weight, eps, holder):
        from aspec_b200.ops import elementwise_sm100 as E
        y, rstd = E.rmsnorm_fwd(x2d, weight, eps)
        ctx.save_for_backward(x2d, weight, rstd)
        ctx.holder = holder
        return y

    @staticmethod
    def backward(ctx, dy):
        from aspec_b200.ops import elementwise_sm100 as E
        x2d, weight, rstd = ctx.saved_tensors
        dx, dw = E.rmsnorm_bwd(dy.contiguous(), x2d, weight, rstd)
        holder = ctx.holder
        main = getattr(holder, "main_grad", None) if holder is not None else None
        if main is not None:
            main.add_(dw)
            holder.main_grad_touched = True
            dw = None
        else:
            dw = dw.to(weight.dtype)
        return dx, dw, None, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        lead = x.shape
        x2d = x.reshape(-1, lead[-1]).contiguous()
        if x2d.shape[0] == 0:
            return x
        holder = weight if isinstance(weight, torch.nn.Parameter) else None
        return _RMSNormFn.apply(x2d, weight, eps, holder).view(lead)
    return rmsnorm_reference(x, weight, eps)


class RMSNorm(torch.nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return rmsnorm(x, self.weight, self.eps)
