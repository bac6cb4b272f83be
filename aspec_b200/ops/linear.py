"""Linear layers on the tcgen05 GEMM (forward, input gradient, weight gradient).

On CUDA bf16 tensors all three products run on ``ops.gemm`` without transposed copies.  If the
weight carries a ``main_grad`` attribute (an fp32 tensor of the weight's shape, owned by the
optimizer) the weight-gradient GEMM accumulates straight into it in fp32 and no bf16 gradient is
materialised: gradient accumulation over micro-batches and the bf16->fp32 gradient copy of the
reference optimizer (aspec/training/optimizer.py:88-147) collapse into the GEMM epilogue.
On CPU tensors this is ``torch.nn.functional.linear`` (the oracle path); on a GPU a bf16 product never leaves the
kernel path (odd shapes are padded, see :func:`linear`).
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


def _pad_dim(t: torch.Tensor, dim: int, mult: int = 8) -> torch.Tensor:
    n = t.shape[dim]
    if n % mult == 0:
        return t
    pad = [0, 0] * t.dim()
    pad[2 * (t.dim() - 1 - dim) + 1] = mult - n % mult
    return F.pad(t, pad)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)``; ``w`` is ``[out, in]``.

    Every bf16 product on a GPU runs on the tcgen05 GEMM: a dimension that is not a multiple of 8 (the TMA row
    alignment) is zero-padded for the call and the result sliced, a bias is added to the kernel's output.  There is
    no library GEMM behind this function for bf16 CUDA tensors; other dtypes on a GPU (fp32 router gates) and all
    CPU tensors use ``torch.nn.functional.linear``.
    """
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if x.shape[-1] != w.shape[1]:
            raise ValueError(f"linear: input width {x.shape[-1]} does not match the weight's {w.shape[1]}")
        lead = x.shape[:-1]
        out_f = w.shape[0]
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.shape[0] == 0:
            return x.new_zeros(*lead, out_f)
        padded = not _kernel_ok(x, w)
        if padded:
            # rare shapes (a 1-wide confidence head, an odd rank): pad to the kernel's alignment for this call;
            # autograd slices the gradients back
            w = _pad_dim(_pad_dim(w, 0), 1).contiguous()
            x2d = _pad_dim(x2d, 1)
        if x2d.stride(1) != 1 or x2d.stride(0) % 8 or x2d.data_ptr() % 16:
            x2d = x2d.contiguous()
        note("gemm", "tcgen05_tma_persistent")
        y = _LinearFn.apply(x2d, w, w if (isinstance(w, torch.nn.Parameter) and not padded) else None)
        if padded:
            y = y[:, :out_f]
        if bias is not None:
            y = y + bias.to(y.dtype)
        return y.reshape(*lead, out_f)
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
