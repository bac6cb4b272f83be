"""EAGLE4 training wrapper: EAGLE3's test-time-training objective in the ``draft`` stage; in the ``candidate_head``
stage a forward KL from the frozen draft's top-k distribution to the low-rank retrieval head, with recall and
captured-mass metrics (reference: aspec/models/eagle4.py:20-38, aspec/models/ops/eagle4_candidate.py:26-54).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from aspec_b200.models.eagle3 import Eagle3Model
from aspec_b200.ops.norm import rmsnorm


def candidate_retrieval_terms(hidden, full_head, down, up, *, teacher_top_k: int, num_candidates: int, chunk_size: int = 128):
    """``(kl_sum, top1_recall_sum, rows, captured_mass_sum)`` over ``hidden [N, D]`` (detached).

    The teacher is the exact head's softmax restricted to its own top ``teacher_top_k``; the student is the full
    low-rank softmax.  Work is chunked so no ``[N, V]`` tensor outlives a chunk (recomputed in backward).
    """
    h = hidden.detach().reshape(-1, hidden.shape[-1])
    if type(chunk_size) is not int or chunk_size <= 0:
        raise ValueError("Candidate loss chunk size must be positive")
    V = full_head.shape[0]
    if not (0 < teacher_top_k <= V and 0 < num_candidates <= V):
        raise ValueError("Candidate counts exceed vocabulary")

    def chunk(states, down_w, up_w):
        with torch.no_grad():
            logits = F.linear(states, full_head.to(states.dtype)).float()
            top, teacher_ids = logits.topk(teacher_top_k, -1)
            teacher_p = torch.softmax(top, -1)
        scores = F.linear(F.linear(states, down_w.to(states.dtype)), up_w.to(states.dtype)).float()
        log_q = scores.log_softmax(-1).gather(-1, teacher_ids)
        loss = (teacher_p * (teacher_p.clamp_min(torch.finfo(torch.float32).tiny).log() - log_q)).sum()
        with torch.no_grad():
            cands = scores.topk(num_candidates, -1).indices
            recall = (cands == teacher_ids[:, :1]).any(-1).float().sum()
            mass = (logits.gather(-1, cands) - logits.logsumexp(-1, keepdim=True)).exp().sum()
        return loss, recall, mass

    total = (down.sum() + up.sum()).float() * 0.0
    recall = total.detach().clone()
    mass = recall.clone()
    for states in h.split(chunk_size):
        vals = checkpoint(chunk, states, down, up, use_reentrant=False) if torch.is_grad_enabled() else chunk(states, down, up)
        total, recall, mass = total + vals[0], recall + vals[1], mass + vals[2]
    return total, recall, torch.tensor(float(h.shape[0]), device=h.device), mass


class Eagle4TrainingModel(Eagle3Model):
    @property
    def uses_target_distribution(self) -> bool:
        return not self.draft_model.candidate_stage

    def _depth_loss(self, hidden, rows, teacher_rows, target):
        draft = self.draft_model
        if not draft.candidate_stage:
            return super()._depth_loss(hidden, rows, teacher_rows, target)
        with torch.no_grad():
            norm_w, _, eps = draft.get_lm_head_params()
            states = rmsnorm(hidden[rows].detach(), norm_w, eps)
        p = draft.eagle4_policy
        kl, recall, _n, mass = candidate_retrieval_terms(
            states, draft.lm_head.weight, draft.efficient_lm_head_down_proj.weight, draft.efficient_lm_head.weight,
            teacher_top_k=p["teacher_top_k"], num_candidates=p["num_candidates"], chunk_size=p["loss_chunk_size"])
        self._candidate_mass = getattr(self, "_candidate_mass", 0.0) + mass.detach()
        return kl, recall, kl.new_zeros(())

    def forward(self, input_ids, hidden_states_list, loss_mask, *args, **kwargs):
        draft = self.draft_model
        self._candidate_mass = torch.zeros((), device=input_ids.device)
        out = super().forward(input_ids, hidden_states_list, loss_mask, *args, **kwargs)
        if draft.candidate_stage:
            comps = dict(out[5])
            count = out[4].sum()
            comps["candidate_recall"] = ((out[3] * out[4]).sum(), count)
            comps["candidate_mass"] = (self._candidate_mass, count)
            out = out[:5] + (comps,) + out[6:]
        return out
