"""Linear layers on the tcgen05 GEMM (forward, input gradient, weight gradient).

On CUDA bf16 tensors all three products run on ``ops.gemm`` without transposed copies.  If the
weight carries a ``main_grad`` attribute (an fp32 tensor of the weight's shape, owned by the
optimizer) the weight-gradient GEMM accumulates straight into it in fp32 and no bf16 gradient is
materialised: gradient accumulation over micro-batches and the bf16->fp32 gradient copy of the
reference optimizer (aspec/training/optimizer.py:88-147) collapse into the GEMM epilogue.
On CPU tensors this is ``torch.nn.functional.linear`` (the oracle path).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from aspec_b200.ops.observed import note


def _kernel_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, w, w_holder):
        from aspec_b200.ops import gemm as G
        ctx.save_for_backward(x2d, w)
        ctx.w_holder = w_holder
        return G.gemm(x2d, w)

    @staticmethod
    def backward(ctx, dy):
        from aspec_b200.ops import gemm as G
        x2d, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dy, w, b_t=True)
        if ctx.needs_input_grad[1]:
            holder = ctx.w_holder
            main = getattr(holder, "main_grad", None) if holder is not None else None
            if main is not None:
                G.gemm(dy, x2d, a_t=True, b_t=True, out=main, addend=main, out_dtype=torch.float32)
                holder.main_grad_touched = True
            else:
                dw = G.gemm(dy, x2d, a_t=True, b_t=True)
        return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)``; ``w`` is ``[out, in]``."""
    if bias is None and _kernel_ok(x, w) and x.shape[-1] == w.shape[1]:
        lead = x.shape[:-1]
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.stride(1) != 1 or x2d.stride(0) % 8 or x2d.data_ptr() % 16:
            x2d = x2d.contiguous()
        if x2d.shape[0] == 0:
            return x.new_zeros(*lead, w.shape[0])
        note("gemm", "tcgen05_tma_persistent")
        y = _LinearFn.apply(x2d, w, w if isinstance(w, torch.nn.Parameter) else None)
        return y.view(*lead, w.shape[0])
    note("gemm", "torch")
    return F.linear(x, w, bias)


class Linear(torch.nn.Module):
    """Bias-free (by default) linear layer backed by :func:`linear`."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = torch.nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.weight.device.type != "meta":
            torch.nn.init.normal_(self.weight, mean=0.0, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
