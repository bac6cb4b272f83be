"""Several named ``nn.Parameter``s stored back to back so one GEMM can use them as one weight.

``k_proj.weight`` / ``v_proj.weight`` (and ``gate_proj`` / ``up_proj``) keep their individual names in
``state_dict`` - checkpoints and exports look exactly like the reference's - but they are views of
one contiguous allocation, so the kernel path runs a single ``[sum(out_i), in]`` GEMM.  When an
optimizer re-homes parameters into its flat buffers it keeps module order, which preserves the
adjacency; ``fused_weight`` re-derives the fused view from the first parameter's storage and falls
back to ``torch.cat`` (autograd-visible, used on the CPU oracle path) when they are not adjacent.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from aspec_b200.ops.linear import _kernel_ok


def allocate_adjacent(shapes: Sequence[Sequence[int]], device=None, dtype=None) -> List[torch.nn.Parameter]:
    total = sum(int(torch.Size(s).numel()) for s in shapes)
    flat = torch.empty(total, device=device, dtype=dtype)
    out, off = [], 0
    for s in shapes:
        n = int(torch.Size(s).numel())
        out.append(torch.nn.Parameter(flat[off:off + n].view(*s)))
        off += n
    return out


def _adjacent(params: Sequence[torch.Tensor]) -> bool:
    if any(not p.is_contiguous() for p in params):
        return False
    esz = params[0].element_size()
    storage = params[0].untyped_storage().data_ptr()
    for a, b in zip(params[:-1], params[1:]):
        if a.data_ptr() + a.numel() * esz != b.data_ptr() or a.dtype != b.dtype:
            return False
        # separately allocated tensors can be neighbours in the allocator's block by chance: the fused view needs one storage
        if b.untyped_storage().data_ptr() != storage:
            return False
    return True


def _span(first: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    return first.detach().as_strided((rows, cols), (cols, 1), first.storage_offset())


class _FusedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, fused_w, *params):
        from aspec_b200.ops import gemm as G
        ctx.save_for_backward(x2d, fused_w)
        ctx.params = params
        return G.gemm(x2d, fused_w)

    @staticmethod
    def backward(ctx, dy):
        from aspec_b200.ops import gemm as G
        x2d, fused_w = ctx.saved_tensors
        params = ctx.params
        dy = dy.contiguous()
        dx = G.gemm(dy, fused_w, b_t=True) if ctx.needs_input_grad[0] else None
        grads = [None] * len(params)
        if any(ctx.needs_input_grad[2:]):
            mains = [getattr(p, "main_grad", None) for p in params]
            if all(m is not None for m in mains) and _adjacent(mains):
                fused_main = _span(mains[0], fused_w.shape[0], fused_w.shape[1])
                G.gemm(dy, x2d, a_t=True, b_t=True, out=fused_main, addend=fused_main,
                       out_dtype=torch.float32)
                for p in params:
                    p.main_grad_touched = True
            else:
                dw = G.gemm(dy, x2d, a_t=True, b_t=True)
                off = 0
                for i, p in enumerate(params):
                    g = dw[off:off + p.shape[0]]
                    off += p.shape[0]
                    m = mains[i]
                    if m is not None:
                        m.add_(g)
                        p.main_grad_touched = True
                    else:
                        grads[i] = g
        return (dx, None, *grads)


def fused_linear(x: torch.Tensor, params: Sequence[torch.nn.Parameter]) -> torch.Tensor:
    """``x @ cat(params, 0).T`` as one GEMM (all ``params`` are ``[out_i, in]``)."""
    cols = params[0].shape[1]
    rows = sum(p.shape[0] for p in params)
    if x.is_cuda and _adjacent(params) and _kernel_ok(x, params[0]) and rows % 8 == 0:
        fused = _span(params[0], rows, cols)
        lead = x.shape[:-1]
        x2d = x.reshape(-1, cols)
        if x2d.stride(1) != 1 or x2d.stride(0) % 8 or x2d.data_ptr() % 16:
            x2d = x2d.contiguous()
        if x2d.shape[0] == 0:
            return x.new_zeros(*lead, rows)
        return _FusedLinearFn.apply(x2d, fused, *params).view(*lead, rows)
    return torch.nn.functional.linear(x, torch.cat(list(params), 0))
