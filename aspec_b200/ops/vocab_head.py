"""Vocabulary head + selective loss for block-drafting objectives.

Computes, for ``R`` supervised draft rows,

    logits  = hidden @ W_lm^T  (+ prev_emb @ W_markov2^T)            [R, V]
    teacher = teacher_hidden[t_index] @ W_lm^T                       (frozen)
    ce      = cross_entropy(logits, label)
    l1      = sum_v |softmax(logits) - softmax(teacher)|

and the weighted numerators ``sum(w * ce)``, ``sum(w * l1)`` that the DSpark / DFlash wrappers pool
(reference: aspec/models/dspark.py:553-636, aspec/models/ops/tiled_l1.py, aspec/models/ops/loss.py).

CUDA path: two tcgen05 GEMMs whose epilogue emits bf16 logits plus per-tile softmax partials
(max, sum-exp); one streaming kernel that turns both logit matrices into per-row CE / L1 /
accuracy and overwrites the student logits with d(loss)/d(logits); the backward is then three
GEMMs (hidden, Markov embedding, Markov projection).  The teacher projection runs over the unique
context rows when that is fewer rows than the supervised set (short documents), which is the
reference's "context teacher projection" reuse (aspec/models/dspark.py:377-420).
No [R, V] fp32 tensor is ever materialised.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def head_loss_reference(hidden, lm_w, labels, weight, *, prev_emb=None, markov_w2=None,
                        teacher_hidden=None, t_index=None, a_ce=1.0, a_l1=0.0, mode=0, teacher_w=None):
    """fp32 PyTorch statement of the op.  Returns (numerator, ce[R], l1[R], correct[R])."""
    logits = F.linear(hidden.float(), lm_w.float())
    if prev_emb is not None:
        logits = logits + F.linear(prev_emb.float(), markov_w2.float())
    R = logits.shape[0]
    l1 = logits.new_zeros(R)
    tw = lm_w if teacher_w is None else teacher_w
    if mode == 1:
        t = F.linear(teacher_hidden.float(), tw.float())
        if t_index is not None:
            t = t[t_index.long()]
        q = torch.softmax(t, -1)
        ce = torch.logsumexp(logits, -1) - (q * logits).sum(-1)
        labels = t.argmax(-1)
    else:
        ce = F.cross_entropy(logits, labels.long(), reduction="none") if R else logits.new_zeros(0)
        if teacher_hidden is not None:
            t = F.linear(teacher_hidden.float(), tw.float())
            if t_index is not None:
                t = t[t_index.long()]
            l1 = (torch.softmax(logits, -1) - torch.softmax(t, -1)).abs().sum(-1)
    correct = (logits.argmax(-1) == labels.long()).float() if R else logits.new_zeros(0)
    num = (weight.float() * (a_ce * ce + a_l1 * l1)).sum()
    return num, ce.detach(), l1.detach(), correct


class _HeadLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, lm_w, prev_emb, markov_w2, teacher_hidden, t_index, labels, weight,
                a_ce, a_l1, mode, w2_holder, teacher_w, lm_holder):
        from aspec_b200.ops import elementwise_sm100 as E
        from aspec_b200.ops import gemm as G
        R, D = hidden.shape
        V = lm_w.shape[0]
        dev = hidden.device
        nt = (V + G.TILE_N - 1) // G.TILE_N
        need_grad = any(ctx.needs_input_grad[i] for i in (0, 1, 2, 3))
        stats = torch.empty(nt, R, 2, dtype=torch.float32, device=dev)
        logits = torch.empty(R, V, dtype=torch.bfloat16, device=dev)
        G.gemm(hidden, lm_w, a2=prev_emb, b2=markov_w2, out=logits, epilogue=G.EPI_ROWSTATS, stats=stats)
        lse_s = E.merge_rowstats(stats)
        t_logits = lse_t = None
        if teacher_hidden is not None:
            Tt = teacher_hidden.shape[0]
            t_stats = torch.empty(nt, Tt, 2, dtype=torch.float32, device=dev)
            t_logits = torch.empty(Tt, V, dtype=torch.bfloat16, device=dev)
            G.gemm(teacher_hidden, lm_w if teacher_w is None else teacher_w, out=t_logits,
                   epilogue=G.EPI_ROWSTATS, stats=t_stats)
            lse_t = E.merge_rowstats(t_stats)
        ce, l1, correct = E.vocab_loss(logits, t_logits, lse_s, lse_t, t_index, labels, weight,
                                       mode=mode, a_ce=a_ce, a_l1=a_l1, write_grad=need_grad)
        num = (weight * (a_ce * ce + a_l1 * l1)).sum()
        ctx.save_for_backward(logits if need_grad else None, hidden, lm_w, prev_emb, markov_w2)
        ctx.w2_holder = w2_holder
        ctx.lm_holder = lm_holder
        ctx.mark_non_differentiable(ce, l1, correct)
        return num, ce, l1, correct

    @staticmethod
    def backward(ctx, dnum, _dce, _dl1, _dcorrect):
        from aspec_b200.ops import elementwise_sm100 as E
        from aspec_b200.ops import gemm as G
        dlogits, hidden, lm_w, prev_emb, markov_w2 = ctx.saved_tensors
        scale = dnum.float().reshape(1)
        dhidden = dprev = dw2 = dlm = None
        if ctx.needs_input_grad[1]:       # trainable student head (EAGLE): dW = dlogits^T hidden
            holder = ctx.lm_holder
            main = getattr(holder, "main_grad", None) if holder is not None else None
            g = G.gemm(dlogits, hidden, a_t=True, b_t=True, out_dtype=torch.float32)
            g.mul_(scale)
            if main is not None:
                main.add_(g)
                holder.main_grad_touched = True
            else:
                dlm = g.to(lm_w.dtype)
        if ctx.needs_input_grad[0]:
            acc = G.gemm(dlogits, lm_w, b_t=True, out_dtype=torch.float32)
            dhidden = E.cast_scale(acc, scale)
        if prev_emb is not None and ctx.needs_input_grad[2]:
            acc = G.gemm(dlogits, markov_w2, b_t=True, out_dtype=torch.float32)
            dprev = E.cast_scale(acc, scale)
        if prev_emb is not None and ctx.needs_input_grad[3]:
            holder = ctx.w2_holder
            main = getattr(holder, "main_grad", None) if holder is not None else None
            g = G.gemm(dlogits, prev_emb, a_t=True, b_t=True, out_dtype=torch.float32)
            g.mul_(scale)
            if main is not None:
                main.add_(g)
                holder.main_grad_touched = True
            else:
                dw2 = g.to(markov_w2.dtype)
        return dhidden, dlm, dprev, dw2, None, None, None, None, None, None, None, None, None, None


def head_loss(hidden: torch.Tensor, lm_w: torch.Tensor, labels: torch.Tensor, weight: torch.Tensor, *,
              prev_emb: Optional[torch.Tensor] = None, markov_w2: Optional[torch.Tensor] = None,
              teacher_hidden: Optional[torch.Tensor] = None, t_index: Optional[torch.Tensor] = None,
              a_ce: float = 1.0, a_l1: float = 0.0, mode: int = 0, teacher_w: Optional[torch.Tensor] = None,
              chunk_rows: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Weighted loss numerator plus detached per-row ``ce``, ``l1`` and ``correct``.

    ``chunk_rows > 0`` bounds the vocabulary-sized intermediates: rows are processed ``chunk_rows`` at a time and each
    chunk's logits are recomputed in its backward instead of being kept (what the reference does per anchor-sized chunk of
    a packed row under activation checkpointing, aspec/models/dspark.py:339-483).  Peak memory is then two
    ``[chunk_rows, V]`` bf16 matrices whatever the row's number of blocks; a call with no more rows than that is
    unchanged.

    ``hidden [R, D]``; ``lm_w [V, D]`` frozen; ``labels [R]`` int64; ``weight [R]`` fp32 (0 for rows
    that are not supervised); ``prev_emb [R, r]`` with ``markov_w2 [V, r]`` adds the Markov bias;
    ``teacher_hidden [Tt, D]`` rows are selected per supervised row by ``t_index [R]`` (int32) and projected
    with ``teacher_w`` (default ``lm_w``).  ``mode=1`` is the EAGLE soft-target cross entropy
    ``logsumexp(z) - sum_v softmax(teacher)_v z_v``; there ``correct`` compares the two arg-maxima and
    ``lm_w`` may be a trainable parameter.
    """
    if chunk_rows and hidden.shape[0] > chunk_rows:
        return _chunked_head_loss(hidden, lm_w, labels, weight, int(chunk_rows), prev_emb=prev_emb, markov_w2=markov_w2,
                                  teacher_hidden=teacher_hidden, t_index=t_index, a_ce=a_ce, a_l1=a_l1, mode=mode,
                                  teacher_w=teacher_w)
    use_kernel = (hidden.is_cuda and hidden.dtype == torch.bfloat16 and lm_w.dtype == torch.bfloat16
                  and lm_w.shape[0] % 8 == 0 and hidden.shape[1] % 8 == 0 and hidden.shape[0] > 0)
    if (not use_kernel and hidden.is_cuda and hidden.dtype == torch.bfloat16 and lm_w.dtype == torch.bfloat16
            and hidden.shape[0] > 0):
        # on a GPU the fused head is the only bf16 path: refuse the shape rather than run the fp32 statement silently
        raise ValueError(f"vocabulary head kernel needs vocab and hidden sizes that are multiples of 8, got "
                         f"{tuple(lm_w.shape)}; pad the head (and mask the padded logits) or run in fp32")
    if not use_kernel:
        return head_loss_reference(hidden, lm_w, labels, weight, prev_emb=prev_emb, markov_w2=markov_w2,
                                   teacher_hidden=teacher_hidden, t_index=t_index, a_ce=a_ce, a_l1=a_l1,
                                   mode=mode, teacher_w=teacher_w)
    if teacher_hidden is not None and t_index is None:
        t_index = torch.arange(hidden.shape[0], device=hidden.device, dtype=torch.int32)
    holder = markov_w2 if isinstance(markov_w2, torch.nn.Parameter) else None
    return _HeadLossFn.apply(
        hidden.contiguous(), lm_w, prev_emb.contiguous() if prev_emb is not None else None, markov_w2,
        teacher_hidden.contiguous() if teacher_hidden is not None else None,
        t_index.to(torch.int32).contiguous() if t_index is not None else None,
        labels.long().contiguous(), weight.float().contiguous(), float(a_ce), float(a_l1), int(mode), holder,
        teacher_w, lm_w if isinstance(lm_w, torch.nn.Parameter) else None)


def _chunked_head_loss(hidden, lm_w, labels, weight, chunk_rows, *, prev_emb, markov_w2, teacher_hidden, t_index, a_ce, a_l1,
                       mode, teacher_w):
    """Row chunks of the head, each under activation checkpointing.  A chunk brings its own teacher rows (gathered by
    ``t_index``, so rows shared between chunks are projected once per chunk that uses them) - no host synchronisation."""
    from torch.utils.checkpoint import checkpoint
    R = hidden.shape[0]
    recompute = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (hidden, lm_w, prev_emb, markov_w2))

    def one(h, lab, wgt, prev, teach):
        return head_loss(h, lm_w, lab, wgt, prev_emb=prev, markov_w2=markov_w2, teacher_hidden=teach, t_index=None,
                         a_ce=a_ce, a_l1=a_l1, mode=mode, teacher_w=teacher_w)

    nums, ces, l1s, oks = [], [], [], []
    for s in range(0, R, chunk_rows):
        sl = slice(s, min(s + chunk_rows, R))
        teach = None
        if teacher_hidden is not None:
            teach = teacher_hidden[sl] if t_index is None else teacher_hidden.index_select(0, t_index[sl].long())
        args = (hidden[sl], labels[sl], weight[sl], prev_emb[sl] if prev_emb is not None else None, teach)
        num, ce, l1, ok = checkpoint(one, *args, use_reentrant=False) if recompute else one(*args)
        nums.append(num)
        ces.append(ce.detach())
        l1s.append(l1.detach())
        oks.append(ok.detach())
    return torch.stack(nums).sum(), torch.cat(ces), torch.cat(l1s), torch.cat(oks)
