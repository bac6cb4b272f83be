"""DSpark training wrapper: DFlash backbone + Markov-biased head + CE / L1 / confidence losses.

Objective (reference: aspec/models/dspark.py:174-636):

* slot ``j`` predicts token ``anchor + j + 1``; a label is valid when in bounds and in the anchor's
  document; ``eval = cumprod_j(keep & valid & loss_mask[label])`` so the first gap ends the block;
  weight ``w = eval * exp(-j / gamma)`` (gamma 4), denominator ``sum(w)``;
* ``logits = hidden @ W_lm^T + markov_w2(markov_w1(prev))`` with ``prev_0`` the anchor token and
  ``prev_j = label_{j-1}``;
* teacher distribution = frozen head on the Target's last hidden state at ``label - 1``;
  ``L1 = sum_v |softmax(logits) - softmax(teacher)|``; ``accept = clamp(1 - L1 / 2, 0, 1)``;
* ``numerator = a_ce * sum(w * CE) + a_l1 * sum(w * L1) + a_conf * sum(w * BCE(conf, accept))`` plus
  MoE / sparse-indexer terms.

The vocabulary-sized work is one fused op (``ops.vocab_head.head_loss``): no fp32 ``[rows, V]`` tensor
exists and nothing is recomputed under activation checkpointing.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from aspec_b200.models.dflash import DFlashModel
from aspec_b200.ops.acceptance import acceptance_components, acceptance_statistics
from aspec_b200.ops.vocab_head import head_loss


class DSparkModel(DFlashModel):
    prediction_start = 0

    def __init__(self, draft_model, block_size: int = 7, num_anchors: int = 512,
                 loss_decay_gamma: float = 4.0, ce_loss_alpha: float = 0.1, l1_loss_alpha: float = 0.9,
                 confidence_head_alpha: float = 1.0, attention_backend: str = "sm100_flash",
                 draft_context_parallel_size: int = 1, deterministic_anchor_sampling: bool = False,
                 anchor_seed: int = 0, anchor_sampling_scope: str = "row",
                 l1_target_sampling=(1.0, 1.0, -1), l1_draft_sampling=(1.0, 1.0, -1)):
        super().__init__(draft_model=draft_model, block_size=block_size, num_anchors=num_anchors,
                         loss_objective="decay", dpace_alpha=0.5, loss_decay_gamma=loss_decay_gamma,
                         attention_backend=attention_backend,
                         draft_context_parallel_size=draft_context_parallel_size,
                         deterministic_anchor_sampling=deterministic_anchor_sampling,
                         anchor_seed=anchor_seed, anchor_sampling_scope=anchor_sampling_scope)
        self.ce_loss_alpha = float(ce_loss_alpha)
        self.l1_loss_alpha = float(l1_loss_alpha)
        self.confidence_head_alpha = float(confidence_head_alpha)
        self.l1_sampling = (tuple(l1_target_sampling), tuple(l1_draft_sampling))
        self.l1_sampling_enabled = self.l1_sampling != ((1.0, 1.0, -1), (1.0, 1.0, -1))

    @property
    def uses_target_distribution(self) -> bool:
        if self._indexer_warmup_kind() is not None:
            return False
        return self.l1_loss_alpha > 0 or (
            self.draft_model.confidence_head is not None and self.confidence_head_alpha > 0)

    def forward(self, input_ids, hidden_states_list, loss_mask, lm_head_weight,
                last_hidden_states=None, ctx_doc_ids=None, base_position_ids=None,
                packed_context_positions=None, injected_anchors=None, injected_keep_mask=None,
                anchor_seed=None, packed_document_lengths=None, attention_mask=None, draft_prefix=None):
        B, T = input_ids.shape
        dev = input_ids.device
        bs = self.block_size
        aux: dict = {"router_logits": [], "csa_losses": [], "qsa_losses": [], "dsa_losses": [],
                     "block_size": self.block_size}
        draft_prefix = self._prepare_draft_prefix(input_ids, last_hidden_states, attention_mask, draft_prefix,
                                                  ctx_doc_ids, base_position_ids, packed_document_lengths)
        hidden, layout, keep = self._draft_backbone(
            input_ids, hidden_states_list, loss_mask, ctx_doc_ids=ctx_doc_ids,
            base_position_ids=base_position_ids, injected_anchors=injected_anchors,
            injected_keep_mask=injected_keep_mask, anchor_seed=anchor_seed,
            packed_document_lengths=packed_document_lengths, attention_mask=attention_mask, aux=aux,
            draft_prefix=draft_prefix)
        n = layout.n
        j = torch.arange(bs, device=dev)[None]
        label = layout.anchor[:, None] + j + 1                                   # [n, bs]
        valid = label < T
        safe = label.clamp(max=T - 1)
        flat_label = layout.row[:, None] * T + safe
        if ctx_doc_ids is not None:
            docs = ctx_doc_ids.reshape(-1)
            valid = valid & (docs[flat_label] == docs[layout.flat_anchor][:, None])
        safe = torch.where(keep[:, None], safe, torch.zeros_like(safe))
        flat_label = layout.row[:, None] * T + safe
        eval_b = keep[:, None] & valid & (loss_mask.reshape(-1)[flat_label] > 0.5)
        eval_mask = eval_b.to(torch.int32).cumprod(-1).float()
        eval_mask = eval_mask * (j >= self.prediction_start)
        w = eval_mask * self._decay(dev)[None]
        den = w.sum()

        if self._indexer_warmup_kind() is not None:
            num, comps = self._aux_losses(aux, w, den)
            key = f"{self._indexer_warmup_kind()}_indexer_loss"
            if key not in comps:
                raise RuntimeError(f"{key[:3].upper()} indexer warm-up produced no indexer KL objective")
            zero = hidden.new_zeros((), dtype=torch.float32)
            pp = hidden.new_zeros(bs, dtype=torch.float32)
            return num / den.clamp(min=1e-6), zero, pp, pp.clone(), pp.clone(), comps, (num, den.detach())

        ids = input_ids.reshape(-1)
        target_ids = ids[flat_label]
        anchor_tok = ids[layout.flat_anchor]
        prev_ids = torch.cat([anchor_tok[:, None], target_ids[:, :-1]], -1)
        teacher_hidden = t_index = None
        if self.uses_target_distribution:
            if last_hidden_states is None:
                raise ValueError("DSpark L1/confidence losses require target last_hidden_states; set "
                                 "inference.store_last_hidden_states=true in the run config.")
            t_flat = (layout.row[:, None] * T + (safe - 1).clamp(min=0)).reshape(-1)
            teacher_hidden, t_index = self._teacher_rows(last_hidden_states, t_flat, layout)

        markov = self.draft_model.markov_head
        prev_emb = markov.get_prev_embeddings(prev_ids.reshape(-1)).to(hidden.dtype) if markov is not None else None
        sampled = self.l1_sampling_enabled and teacher_hidden is not None
        head_kw = dict(prev_emb=prev_emb, markov_w2=markov.markov_w2.weight if markov is not None else None,
                       teacher_hidden=None if sampled else teacher_hidden, t_index=None if sampled else t_index,
                       a_ce=self.ce_loss_alpha,
                       a_l1=self.l1_loss_alpha if (teacher_hidden is not None and not sampled) else 0.0)
        vp = getattr(self, "vocab_parallel", None)
        if vp is not None and sampled:
            raise NotImplementedError("dspark_l1_* sampling transforms need the whole vocabulary on one rank; "
                                      "run with training.vocab_parallel_size=1")
        if vp is not None and hidden.is_cuda:
            # ``lm_head_weight`` is this rank's row shard of the Target head; statistics merge over the peers' memory
            from aspec_b200.parallel.vocab_parallel import vocab_parallel_head_loss
            num_ce_l1, ce, l1, correct = vocab_parallel_head_loss(vp, hidden, lm_head_weight, target_ids.reshape(-1),
                                                                  w.reshape(-1), **head_kw)
        else:
            # a packed row can hold more blocks than one document's anchor budget: the head then runs per
            # anchor-budget-sized chunk, recomputing each chunk's logits in backward
            num_ce_l1, ce, l1, correct = head_loss(hidden, lm_head_weight, target_ids.reshape(-1), w.reshape(-1),
                                                   chunk_rows=self.num_anchors * self.block_size, **head_kw)
        wf = w.reshape(-1)
        if sampled:
            # L1 on the distributions a sampler would draw from (temperature / top-p / top-k): row-chunked logits
            from aspec_b200.ops.loss_sampling import sampled_l1
            rows = teacher_hidden[t_index.long()] if t_index is not None else teacher_hidden
            l1_live = sampled_l1(hidden, lm_head_weight, rows.to(hidden.dtype), prev_emb=prev_emb,
                                 markov_w2=head_kw["markov_w2"], target_sampling=self.l1_sampling[0],
                                 draft_sampling=self.l1_sampling[1])
            num_ce_l1 = num_ce_l1 + self.l1_loss_alpha * (l1_live * wf).sum()
            l1 = l1_live.detach()
        ce_num = (ce * wf).sum()
        l1_num = (l1 * wf).sum() if teacher_hidden is not None else ce_num.new_zeros(())
        conf_num = ce_num.new_zeros(())
        accept = None
        if teacher_hidden is not None:
            accept = (1.0 - 0.5 * l1).clamp(0.0, 1.0)
        if self.draft_model.confidence_head is not None and self.confidence_head_alpha > 0 and accept is not None:
            feats = hidden
            if self.draft_model.confidence_head_with_markov:
                feats = torch.cat([hidden, prev_emb], -1)
            pred = self.draft_model.confidence_head(feats).float()
            conf_num = (F.binary_cross_entropy_with_logits(pred, accept.detach(), reduction="none") * wf).sum()
        num = num_ce_l1 + self.confidence_head_alpha * conf_num
        aux_num, aux_comps = self._aux_losses(aux, w, den)
        num = num + aux_num
        loss = num / den.clamp(min=1e-6)
        d = den.detach()
        comps = {"ce_loss": (ce_num.detach(), d), "l1_loss": (l1_num.detach(), d),
                 "confidence_loss": (conf_num.detach(), d), **aux_comps}
        with torch.no_grad():
            if accept is not None:
                s = self.prediction_start
                stats = F.pad(acceptance_statistics(accept.view(n, bs)[:, s:], eval_mask[:, s:]), (s, 0))
                obs = acceptance_components(stats)
                if self.mtp_conditioning:
                    # the visible first candidate is not a prediction: report the suffix only
                    obs = {("suffix_tau_probabilistic" if k == "tau_probabilistic"
                            else f"suffix_accept_rate@{int(k.split('@')[1]) - s}"): v for k, v in obs.items()
                           if k == "tau_probabilistic" or int(k.split('@')[1]) >= s}
                comps.update(obs)
            correct = correct.view(n, bs) * (eval_mask > 0.5)
            accuracy = correct.sum() / eval_mask.sum().clamp(min=1e-6)
            count_pp = eval_mask.sum(0)
            cpp = count_pp.clamp(min=1.0)
            loss_pp = (ce.view(n, bs) * eval_mask).sum(0) / cpp
            acc_pp = correct.sum(0) / cpp
        return loss, accuracy, loss_pp, acc_pp, count_pp, comps, (num, d)
