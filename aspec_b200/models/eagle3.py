"""EAGLE3 training wrapper: test-time-training recurrence over ``length`` depths on packed tokens.

Semantics (reference: aspec/models/eagle3.py:437-727, aspec/training/eagle3_trainer.py:343-400):

* token ids and the teacher's hidden states are shifted left by one inside each document (the draft at
  position ``t`` consumes token ``t + 1``); at depth ``i`` they are shifted by a further ``i`` and so is the
  loss mask; shifts never cross a document boundary (out-of-document slots are padding, mask 0);
* depth 0 starts from ``fc(features)``, depth ``i`` from the previous depth's output; attention at depth ``i``
  sees the depth-0 keys causally plus one key per earlier depth at the same position;
* per-depth loss over positions whose (shifted) mask is set: forward KL ``logsumexp(z) - sum p z`` against the
  teacher distribution (``lm_head(last_hidden)``, optionally restricted to a pruned draft vocabulary), or
  LK-alpha ``-log sum min(p, q)``, or LK-lambda ``lam * KL + (1 - lam) * TV`` with
  ``lam = exp(-eta * mean alpha)``; depth weights default ``0.8 ** i``.

``forward`` returns the same 7-tuple as the block-drafting wrappers so one trainer drives every algorithm:
the numerator is ``sum_i w_i * loss_sum_i`` with each depth normalised by its own supervised count.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.ops.norm import rmsnorm
from aspec_b200.ops.vocab_head import head_loss


@dataclass
class LazyTarget:
    """Teacher given as hidden states to be projected with the frozen Target head."""
    hidden_states: torch.Tensor            # [T, Dt] post-norm last hidden states
    lm_head_weight: torch.Tensor           # [V, Dt]
    t2d: Optional[torch.Tensor] = None
    pruned_weight: Optional[torch.Tensor] = None


@dataclass
class PrecomputedTarget:
    target_p: torch.Tensor                 # [T, Vd] probabilities
    position_mask: Optional[torch.Tensor] = None


@dataclass
class CachedLogitsTarget:
    target_logits: torch.Tensor            # [T, Vd]


def default_ploss_weights(length: int) -> List[float]:
    return [0.8 ** i for i in range(length)]


def shift_within_documents(values: torch.Tensor, doc_end: torch.Tensor, shift: int, fill=0):
    """``out[t] = values[t + shift]`` if ``t + shift`` is still inside ``t``'s document, else ``fill``."""
    T = values.shape[0]
    t = torch.arange(T, device=values.device)
    src = t + shift
    ok = src < doc_end
    out = values[src.clamp(max=T - 1)]
    mask = ok.view(-1, *([1] * (values.dim() - 1)))
    return torch.where(mask, out, torch.full_like(out, fill)), ok


class Eagle3Model(nn.Module):
    def __init__(self, draft_model, length: int = 7, loss_type: str = "forward_kl", lk_eta: float = 3.0,
                 ploss_weights: Optional[Sequence[float]] = None, attention_backend: str = "sm100_flash",
                 gradient_checkpointing: bool = False):
        super().__init__()
        if loss_type not in ("forward_kl", "lk_alpha", "lk_lambda"):
            raise ValueError("loss_type must be forward_kl, lk_alpha or lk_lambda")
        self.draft_model = draft_model
        self.length = int(length)
        self.loss_type, self.lk_eta = loss_type, float(lk_eta)
        self.ploss_weights = list(ploss_weights) if ploss_weights else default_ploss_weights(self.length)
        if len(self.ploss_weights) != self.length:
            raise ValueError("ploss_weights must have one entry per TTT depth")
        self.attention_backend = attention_backend
        self.gradient_checkpointing = gradient_checkpointing
        self.block_size = self.length          # per-position metrics have one slot per depth

    uses_target_distribution = True
    supports_sequence_parallel = True       # ``sequence_parallel = (rank, size, group)`` + ``draft_model.ulysses``

    # -- per-depth loss ---------------------------------------------------------------------------
    def _depth_loss(self, hidden, rows, teacher_rows, target: LazyTarget):
        """Sum of the loss over the supervised ``rows`` of one depth.  Returns (sum, correct, alpha_sum)."""
        draft = self.draft_model
        norm_w, head_w, eps = draft.get_lm_head_params()
        h = rmsnorm(hidden[rows], norm_w, eps)
        teacher_w = target.lm_head_weight
        if draft.vocab_pruned:
            teacher_w = target.pruned_weight if target.pruned_weight is not None else teacher_w[draft.t2d]
        n = rows.numel()
        ones = torch.ones(n, device=hidden.device)
        if self.loss_type == "forward_kl":
            num, _ce, _l1, correct = head_loss(h, head_w, torch.zeros(n, dtype=torch.long, device=hidden.device), ones,
                                               teacher_hidden=teacher_rows, mode=1, teacher_w=teacher_w)
            return num, correct.sum(), num.new_zeros(())
        logits = F.linear(h.float(), head_w.float())
        t_logits = F.linear(teacher_rows.float(), teacher_w.float())
        tp_tilde = torch.softmax(t_logits, -1)
        q = torch.softmax(logits, -1)
        coverage = 1.0
        if draft.vocab_pruned:
            full = torch.logsumexp(F.linear(teacher_rows.float(), target.lm_head_weight.float()), -1)
            coverage = torch.exp(torch.logsumexp(t_logits, -1) - full)[:, None]
        tp = tp_tilde * coverage
        alpha = torch.minimum(tp, q).sum(-1)
        correct = (logits.argmax(-1) == tp_tilde.argmax(-1)).float().sum()
        if self.loss_type == "lk_alpha":
            return (-torch.log(alpha.clamp(min=1e-8))).sum(), correct, alpha.sum().detach()
        lam = torch.exp(-self.lk_eta * alpha.mean().detach())
        kl = (tp_tilde * (torch.log(tp_tilde.clamp(min=1e-30)) - torch.log_softmax(logits, -1))).sum(-1)
        tv = 0.5 * (tp - q).abs().sum(-1)
        return (lam * kl + (1.0 - lam) * tv).sum(), correct, alpha.sum().detach()

    # -- forward --------------------------------------------------------------------------------------
    def forward(self, input_ids, hidden_states_list, loss_mask, lm_head_weight, last_hidden_states=None,
                ctx_doc_ids=None, base_position_ids=None, packed_document_lengths=None, attention_mask=None, **_unused):
        if last_hidden_states is None:
            raise ValueError("EAGLE3 training needs the Target's last_hidden_states")
        draft = self.draft_model
        sp = getattr(self, "sequence_parallel", None)          # (rank, size, process group) of an Ulysses group
        if sp is not None:
            # every rank of the group receives the whole row; it pads it to a multiple of the group size, keeps its own
            # slice of the token-wise work and meets the others inside the attention exchange
            if input_ids.shape[0] != 1:
                raise ValueError("sequence-parallel EAGLE training takes one packed row per micro-batch")
            pad = (-input_ids.shape[1]) % sp[1]
            if ctx_doc_ids is None:
                ctx_doc_ids = torch.zeros_like(input_ids)
            if pad:
                def padded(x, value):
                    return None if x is None else torch.cat([x, x.new_full((1, pad, *x.shape[2:]), value)], 1)
                feats_in = hidden_states_list if torch.is_tensor(hidden_states_list) else torch.cat(list(hidden_states_list), -1)
                input_ids, loss_mask = padded(input_ids, 0), padded(loss_mask, 0)
                hidden_states_list, last_hidden_states = padded(feats_in, 0), padded(last_hidden_states, 0)
                ctx_doc_ids, base_position_ids = padded(ctx_doc_ids, -1), padded(base_position_ids, 0)
                attention_mask = padded(attention_mask, 0)
        B, T0 = input_ids.shape
        dev = input_ids.device
        ids = input_ids.reshape(-1)
        mask = loss_mask.reshape(-1).float().to(dev)
        feats = hidden_states_list if torch.is_tensor(hidden_states_list) else torch.cat(list(hidden_states_list), -1)
        wdtype = draft.fc.weight.dtype
        feats = feats.reshape(B * T0, -1).to(wdtype)
        teacher = last_hidden_states.reshape(B * T0, -1).to(wdtype)
        T = B * T0
        # document structure of the packed rows
        if ctx_doc_ids is not None:
            doc = ctx_doc_ids.reshape(-1).to(dev) + torch.arange(B, device=dev).repeat_interleave(T0) * (T0 + 1)
            valid = ctx_doc_ids.reshape(-1).to(dev) >= 0
        else:
            doc = torch.arange(B, device=dev).repeat_interleave(T0)
            valid = (attention_mask.reshape(-1).to(dev) > 0) if attention_mask is not None else torch.ones(T, dtype=torch.bool, device=dev)
        t = torch.arange(T, device=dev)
        first = torch.ones(T, dtype=torch.bool, device=dev)
        first[1:] = doc[1:] != doc[:-1]
        doc_start = torch.where(first, t, torch.zeros_like(t)).cummax(0).values
        last = torch.ones(T, dtype=torch.bool, device=dev)
        last[:-1] = doc[1:] != doc[:-1]
        doc_end = torch.where(last, t + 1, torch.full_like(t, T)).flip(0).cummin(0).values.flip(0)
        positions = (base_position_ids.reshape(-1).to(dev) if base_position_ids is not None else t - doc_start).to(torch.int32)
        mask = mask * valid
        if hasattr(draft, "set_valid_rows") and sp is None:
            draft.set_valid_rows(lambda depth: (t + depth + 1 < doc_end) & valid)

        if sp is not None:
            sp_rank, sp_size, sp_group = sp
            T_loc = T // sp_size
            sl = slice(sp_rank * T_loc, (sp_rank + 1) * T_loc)
            if hasattr(draft, "set_valid_rows"):
                draft.set_valid_rows(lambda depth: ((t + depth + 1 < doc_end) & valid)[sl])
        else:
            sl = slice(0, T)
        target = LazyTarget(teacher, lm_head_weight, getattr(draft, "t2d", None) if draft.vocab_pruned else None)
        hidden = draft.project_hidden_states(feats[sl])
        cache = None
        numerator = hidden.new_zeros((), dtype=torch.float32)
        loss_pp, acc_pp, count_pp = [], [], []
        alphas = []
        for i in range(self.length):
            step_ids, _ = shift_within_documents(ids, doc_end, 1 + i)
            step_mask, inside = shift_within_documents(mask, doc_end, i)
            teacher_i, _ = shift_within_documents(teacher, doc_end, 1 + i)
            step_ids, step_mask, teacher_i = step_ids[sl], step_mask[sl], teacher_i[sl]
            embeds = draft.embed_input_ids(step_ids).to(hidden.dtype)
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled() and sp is None:
                from torch.utils.checkpoint import checkpoint
                hidden, cache = checkpoint(draft.backbone, embeds, hidden, positions, i, cache, doc_start, self.length,
                                           use_reentrant=False)
            else:
                hidden, cache = draft.backbone(embeds, hidden, positions, i, cache, doc_start, self.length)
            rows = (step_mask > 0.5).nonzero(as_tuple=False).squeeze(-1)
            count = step_mask.sum()
            if rows.numel():
                loss_sum, correct, alpha_sum = self._depth_loss(hidden, rows, teacher_i[rows], target)
            else:
                loss_sum = hidden.sum() * 0.0
                correct = alpha_sum = loss_sum.detach()
            total_loss = loss_sum.detach()
            if sp is not None:
                # the depth's supervised rows are spread over the group: normalise by the row's count, report the row's sums
                import torch.distributed as dist
                pooled = torch.stack([total_loss.float(), correct.float(), count.float(), alpha_sum.float()])
                dist.all_reduce(pooled, group=sp_group)
                total_loss, correct, count, alpha_sum = pooled.unbind(0)
            numerator = numerator + self.ploss_weights[i] * loss_sum / count.clamp(min=1.0)
            loss_pp.append(total_loss / count.clamp(min=1.0))
            acc_pp.append((correct / count.clamp(min=1.0)).detach())
            count_pp.append(count.detach())
            alphas.append((alpha_sum / count.clamp(min=1.0)).detach())
            hidden = draft.next_depth_hidden(hidden)
        denominator = torch.ones((), device=dev) / (sp[1] if sp is not None else 1)
        loss_pp, acc_pp, count_pp = torch.stack(loss_pp), torch.stack(acc_pp), torch.stack(count_pp)
        accuracy = (acc_pp * count_pp).sum() / count_pp.sum().clamp(min=1.0)
        comps = {}
        if self.loss_type != "forward_kl":
            comps["lk_alpha"] = ((torch.stack(alphas) * count_pp).sum(), count_pp.sum())
        return numerator, accuracy, loss_pp, acc_pp, count_pp, comps, (numerator, denominator)
