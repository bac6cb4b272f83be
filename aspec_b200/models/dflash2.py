"""DFlash2 training wrapper: DFlash block objective on scaled / soft-capped logits plus the candidate-selector
cross-entropy (reference: aspec/models/dflash2.py:31-134).

Per-layer mask policy: ``sliding_attention`` layers are causal inside the block and windowed, ``full_attention``
layers bidirectional, unless the config pins ``is_causal``.  The selector term scores, for positions ``1..B-1``
of each block, the true successor among the unary top-k given the true predecessor; its weights stop at the first
unsupervised position (cumulative product).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from aspec_b200.models.dflash import DFlashModel
from aspec_b200.ops.linear import linear


class DFlash2Model(DFlashModel):
    def __init__(self, *args, selector_loss_alpha: float = 1.0, **kwargs):
        super().__init__(*args, **kwargs)
        selector_loss_alpha = float(selector_loss_alpha)
        if not math.isfinite(selector_loss_alpha) or selector_loss_alpha < 0:
            raise ValueError(f"dflash2_selector_loss_alpha must be non-negative, got {selector_loss_alpha}")
        self.selector_loss_alpha = selector_loss_alpha
        cfg = self.draft_model.config
        if self.block_size != cfg.block_size:
            raise ValueError("DFlash2 training block_size must match its convolution block_size")
        kinds = list(getattr(cfg, "layer_types", None) or ["full_attention"] * cfg.num_hidden_layers)
        if len(kinds) != cfg.num_hidden_layers:
            raise ValueError(f"DFlash2 layer_types must contain one entry per draft layer, got {len(kinds)} "
                             f"for {cfg.num_hidden_layers} layers")
        if not set(kinds) <= {"full_attention", "sliding_attention"}:
            raise ValueError(f"Unsupported DFlash2 layer types: {sorted(set(kinds))}")
        window = getattr(cfg, "sliding_window", None)
        if "sliding_attention" in kinds and (window is None or int(window) < 1):
            raise ValueError("DFlash2 sliding_attention layers require an explicit positive sliding_window")
        pinned = getattr(cfg, "is_causal", None)
        self.layer_block_mask_options = [
            {"is_causal": (k == "sliding_attention") if pinned is None else bool(pinned),
             "sliding_window": int(window) if k == "sliding_attention" else None} for k in kinds]
        self.attention_is_causal = self.layer_block_mask_options[0]["is_causal"]
        self.sliding_window = self.layer_block_mask_options[0]["sliding_window"]

    def _block_causal(self, layer: int) -> bool:
        return self.layer_block_mask_options[layer]["is_causal"]

    def _compute_logits(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor) -> torch.Tensor:
        cfg = self.draft_model.config
        logits = linear(hidden, lm_head_weight.to(hidden.dtype)).float() * cfg.output_multiplier
        cap = cfg.final_logit_softcapping
        return torch.tanh(logits / cap) * cap if cap is not None and cap > 0 else logits

    def forward(self, input_ids, hidden_states_list, loss_mask, lm_head_weight, last_hidden_states=None,
                ctx_doc_ids=None, base_position_ids=None, packed_context_positions=None, injected_anchors=None,
                injected_keep_mask=None, anchor_seed=None, packed_document_lengths=None, attention_mask=None,
                draft_prefix=None):
        B, T = input_ids.shape
        dev, bs = input_ids.device, self.block_size
        aux: dict = {"router_logits": [], "block_size": bs}
        hidden, layout, keep = self._draft_backbone(
            input_ids, hidden_states_list, loss_mask, ctx_doc_ids=ctx_doc_ids, base_position_ids=base_position_ids,
            injected_anchors=injected_anchors, injected_keep_mask=injected_keep_mask, anchor_seed=anchor_seed,
            packed_document_lengths=packed_document_lengths, attention_mask=attention_mask, aux=aux)
        n = layout.n
        j = torch.arange(bs, device=dev)[None]
        label = layout.anchor[:, None] + j
        safe = label.clamp(max=T - 1)
        flat_label = layout.row[:, None] * T + safe
        target_ids = input_ids.reshape(-1)[flat_label]
        binary = (keep[:, None].float() * (label < T).float() * (j >= self.prediction_start).float()
                  * loss_mask.reshape(-1)[flat_label].float())
        obj_w = binary * (self._decay(dev)[None] if self.loss_objective == "decay" else 1.0)
        logits = self._compute_logits(hidden, lm_head_weight).view(n, bs, -1)
        ce = F.cross_entropy(logits.reshape(n * bs, -1), target_ids.reshape(-1), reduction="none").view(n, bs)
        num = self.ce_loss_alpha * (ce * obj_w).sum()
        comps = {"ce_loss": ((ce.detach() * obj_w).sum(), obj_w.sum().detach())}
        if self.l1_loss_alpha > 0:
            if last_hidden_states is None:
                raise ValueError("DFlash L1 distillation (l1_loss_alpha > 0) requires target last_hidden_states")
            rows = (layout.row[:, None] * T + (safe - 1).clamp(min=0)).reshape(-1)
            teacher = last_hidden_states.reshape(-1, last_hidden_states.shape[-1])[rows].to(hidden.dtype)
            t_prob = torch.softmax(linear(teacher, lm_head_weight.to(hidden.dtype)).float(), -1)
            l1 = (torch.softmax(logits.reshape(n * bs, -1), -1) - t_prob).abs().sum(-1).view(n, bs)
            num = num + self.l1_loss_alpha * (l1 * obj_w).sum()
            comps["l1_loss"] = ((l1.detach() * obj_w).sum(), obj_w.sum().detach())
        # selector: positions 1..bs-1, true predecessor, weights truncated at the first unsupervised slot
        sel_w = obj_w[:, 1:] * (obj_w[:, 1:] > 0).cumprod(-1)
        scores, cand = self.draft_model.candidate_selector.score_candidates(
            hidden.view(n, bs, -1)[:, 1:], logits[:, 1:], target_ids[:, :-1], training_successor_ids=target_ids[:, 1:])
        truth = (cand == target_ids[:, 1:].unsqueeze(-1)).long().argmax(-1)
        sel_ce = F.cross_entropy(scores.reshape(-1, scores.shape[-1]), truth.reshape(-1), reduction="none").view_as(sel_w)
        sel_num = (sel_ce * sel_w).sum()
        comps["selector_loss"] = (sel_num.detach(), sel_w.sum().detach())
        num = num + self.selector_loss_alpha * sel_num
        den = obj_w.sum()
        aux_num, aux_comps = self._aux_losses(aux, obj_w, den)
        num = num + aux_num
        comps.update(aux_comps)
        with torch.no_grad():
            correct = (logits.argmax(-1) == target_ids).float() * (binary > 0.5)
            accuracy = correct.sum() / binary.sum().clamp(min=1e-6)
            count_pp = binary.sum(0)
            cpp = count_pp.clamp(min=1.0)
            loss_pp = (ce * binary).sum(0) / cpp
            acc_pp = correct.sum(0) / cpp
        return num / den.clamp(min=1e-6), accuracy, loss_pp, acc_pp, count_pp, comps, (num, den.detach())
