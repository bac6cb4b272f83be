"""Native MTP training wrapper: recurrent teacher-forced multi-step prediction on packed documents
(reference: aspec/models/mtp.py:26-136).

For a document of ``n`` tokens, ``steps = min(L, max(0, n - 2))`` and every depth runs on the same valid prefix of
``n - steps - 1`` rows.  Depth ``d`` consumes the Target state (depth 0) or the previous depth's output together
with token ``x[t + d + 1]`` and is supervised with ``x[t + d + 2]`` where the loss mask is set there.  Step
weights are ``beta^k`` normalised (scaled by the largest power when ``beta > 1``).
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from aspec_b200.models.draft.mtp import causal_intervals
from aspec_b200.ops.vocab_head import head_loss


def mtp_step_weights(steps: int, beta: float) -> List[float]:
    raw = [beta ** (k if beta <= 1 else k - steps + 1) for k in range(steps)]
    total = sum(raw)
    return [v / total for v in raw]


def packed_documents(B, T0, dev, ctx_doc_ids=None, attention_mask=None):
    """``(doc_start, doc_end, valid)`` over the flattened ``B * T0`` rows."""
    T = B * T0
    if ctx_doc_ids is not None:
        flat = ctx_doc_ids.reshape(-1).to(dev)
        doc = flat + torch.arange(B, device=dev).repeat_interleave(T0) * (T0 + 1)
        valid = flat >= 0
    else:
        doc = torch.arange(B, device=dev).repeat_interleave(T0)
        valid = (attention_mask.reshape(-1).to(dev) > 0) if attention_mask is not None else torch.ones(T, dtype=torch.bool, device=dev)
    doc = torch.where(valid, doc, torch.full_like(doc, -1) - torch.arange(T, device=dev))
    t = torch.arange(T, device=dev)
    first = torch.ones(T, dtype=torch.bool, device=dev)
    first[1:] = doc[1:] != doc[:-1]
    last = torch.ones(T, dtype=torch.bool, device=dev)
    last[:-1] = first[1:]
    doc_start = torch.where(first, t, torch.zeros_like(t)).cummax(0).values
    doc_end = torch.where(last, t + 1, torch.full_like(t, T)).flip(0).cummin(0).values.flip(0)
    return doc_start, doc_end, valid


class MTPModel(nn.Module):
    uses_target_distribution = False
    uses_target_hidden_states = True

    def __init__(self, draft_model, length: int = 3, step_weight_beta: float = 0.6, gradient_checkpointing: bool = False):
        super().__init__()
        self.draft_model = draft_model
        self.length = int(length)
        self.step_weights = mtp_step_weights(self.length, float(step_weight_beta))
        self.gradient_checkpointing = gradient_checkpointing
        self.block_size = self.length
        self.vocab_pruning = False

    def forward(self, input_ids, hidden_states_list, loss_mask, lm_head_weight=None, last_hidden_states=None,
                ctx_doc_ids=None, base_position_ids=None, attention_mask=None, **_unused):
        draft = self.draft_model
        B, T0 = input_ids.shape
        dev, T = input_ids.device, B * T0
        source = last_hidden_states if last_hidden_states is not None else hidden_states_list
        if not torch.is_tensor(source):
            source = source[-1]
        state = source.reshape(T, -1).detach().to(draft.fc.weight.dtype)
        ids = input_ids.reshape(-1)
        mask = loss_mask.reshape(-1).to(dev)
        doc_start, doc_end, valid = packed_documents(B, T0, dev, ctx_doc_ids, attention_mask)
        t = torch.arange(T, device=dev)
        n = doc_end - doc_start
        steps = torch.clamp(n - 2, min=0, max=self.length)
        in_prefix = valid & (steps > 0) & (t - doc_start < n - steps - 1)
        positions = (t - doc_start).to(torch.int32)
        intervals = causal_intervals(doc_start)
        numerator = state.new_zeros((), dtype=torch.float32)
        loss_pp, acc_pp, count_pp = [], [], []
        for depth in range(self.length):
            step_ids = ids[(t + depth + 1).clamp(max=T - 1)]
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                state = checkpoint(draft.predict, state, step_ids, positions, intervals, use_reentrant=False)
            else:
                state = draft.predict(state, step_ids, positions, intervals)
            label_at = (t + depth + 2).clamp(max=T - 1)
            keep = in_prefix & (depth < steps) & (t + depth + 2 < doc_end) & (mask[label_at] > 0)
            rows = keep.nonzero(as_tuple=False).squeeze(-1)
            count = keep.sum().float()
            if rows.numel():
                num, _ce, _l1, correct = head_loss(state[rows], draft.lm_head.weight, ids[label_at[rows]],
                                                   torch.ones(rows.numel(), device=dev), a_ce=1.0)
                hits = correct.sum()
            else:
                num = state.sum() * 0.0
                hits = num.detach()
            loss_k = num / count.clamp(min=1.0)
            numerator = numerator + self.step_weights[depth] * loss_k
            loss_pp.append(loss_k.detach())
            acc_pp.append((hits / count.clamp(min=1.0)).detach())
            count_pp.append(count.detach())
        loss_pp, acc_pp, count_pp = torch.stack(loss_pp), torch.stack(acc_pp), torch.stack(count_pp)
        accuracy = (acc_pp * count_pp).sum() / count_pp.sum().clamp(min=1.0)
        return numerator, accuracy, loss_pp, acc_pp, count_pp, {}, (numerator, torch.ones((), device=dev))
