"""DFlash training wrapper: anchors -> noise blocks -> Draft backbone -> weighted CE (+L1).

Semantics follow the reference wrapper (aspec/models/dflash.py:134-1248):

* ``A`` anchors per row (or per document) are sampled from supervised positions; block ``a`` is
  ``block_size`` draft tokens whose slot 0 carries the anchor token and whose other slots carry
  ``mask_token_id``; slot ``j`` sits at position ``pos(anchor) + j``;
* a block sees the context strictly before its anchor inside its own document (optionally only the
  last ``context_window`` tokens) and its own block (bidirectional unless configured causal);
* slot ``k >= prediction_start`` predicts token ``anchor + k`` with weight
  ``keep * in_bounds * loss_mask[anchor + k]`` times ``exp(-(k - start) / gamma)`` (or D-PACE weights);
* the wrapper returns the additive ``(numerator, denominator)`` so the trainer can pool over
  micro-batches and ranks before dividing.

The implementation flattens the batch into packed token-major tensors and processes only the kept
blocks.  Anchors may be injected (sampled by the data pipeline on the host); when their keep mask
is a CPU tensor the compaction needs no device synchronisation.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from aspec_b200.config.draft_attention import context_shard_alignment, resolve_attention_policy
from aspec_b200.ops import anchors as A
from aspec_b200.ops.attention import build_block_intervals
from aspec_b200.ops.vocab_head import head_loss

_OBJECTIVES = ("decay", "dpace")


def dpace_position_weights(confidences: torch.Tensor, alpha: float) -> torch.Tensor:
    """D-PACE: suffix sums of cumulative products of smoothed per-position confidences."""
    if not 0.0 <= alpha <= 1.0:
        raise ValueError(f"dflash_dpace_alpha must be in [0, 1], got {alpha}")
    with torch.no_grad():
        smooth = (1.0 - alpha) * confidences.float() + alpha
        prod = torch.cumprod(smooth, dim=-1)
        return torch.flip(torch.cumsum(torch.flip(prod, [-1]), -1), [-1]).to(confidences.dtype)


class BlockLayout:
    """Kept blocks of a micro-batch in packed order (all tensors on the model's device)."""

    def __init__(self, row, anchor, slot, n_rows, seq_len, n_slots):
        self.row, self.anchor, self.slot = row, anchor, slot      # [n] int64 each
        self.n_rows, self.seq_len, self.n_slots = n_rows, seq_len, n_slots
        self.n = int(row.shape[0])
        # [lo, hi) over the flattened context of every position a kept block touches (anchor .. anchor +
        # block_size); known without a device round trip when the anchors came from the host
        self.host_span = None

    @property
    def flat_anchor(self) -> torch.Tensor:
        return self.row * self.seq_len + self.anchor


class DFlashModel(nn.Module):
    prediction_start = 1

    def __init__(self, draft_model, block_size: int = 16, num_anchors: int = 512,
                 loss_objective: str = "decay", dpace_alpha: float = 0.5,
                 loss_decay_gamma: float = 7.0, ce_loss_alpha: float = 1.0,
                 l1_loss_alpha: float = 0.0, attention_backend: str = "sm100_flash",
                 draft_context_parallel_size: int = 1, deterministic_anchor_sampling: bool = False,
                 anchor_seed: int = 0, anchor_sampling_scope: str = "row"):
        super().__init__()
        loss_objective = loss_objective.lower()
        if loss_objective not in _OBJECTIVES:
            raise ValueError(f"Unknown DFlash loss objective {loss_objective!r}; expected one of "
                             + ", ".join(sorted(_OBJECTIVES)))
        if not 0.0 <= dpace_alpha <= 1.0:
            raise ValueError(f"dflash_dpace_alpha must be in [0, 1], got {dpace_alpha}")
        if anchor_sampling_scope not in ("row", "sample"):
            raise ValueError("anchor_sampling_scope must be row or sample")
        self.draft_model = draft_model
        cfg = getattr(draft_model, "config", None)
        self.mtp_conditioning = getattr(cfg, "mtp_conditioning", None)
        self.prediction_start = type(self).prediction_start + int(self.mtp_conditioning is not None)
        self.block_size, self.num_anchors = int(block_size), int(num_anchors)
        self.anchor_sampling_scope = anchor_sampling_scope
        self.deterministic_anchor_sampling = deterministic_anchor_sampling
        self.anchor_seed = int(anchor_seed)
        self.loss_objective, self.dpace_alpha = loss_objective, dpace_alpha
        self.loss_decay_gamma = loss_decay_gamma
        self.ce_loss_alpha, self.l1_loss_alpha = float(ce_loss_alpha), float(l1_loss_alpha)
        self.attention_backend = attention_backend
        self.draft_context_parallel_size = int(draft_context_parallel_size)
        if self.mtp_conditioning and (block_size <= self.prediction_start or loss_objective != "decay"):
            raise ValueError("MTP conditioning requires decay loss and an unknown suffix slot")
        if self.mtp_conditioning and (self.draft_context_parallel_size != 1 or anchor_sampling_scope != "row"):
            raise ValueError("MTP conditioning currently requires CP1 row anchors")
        if self.draft_context_parallel_size > 1 and self.num_anchors % self.draft_context_parallel_size:
            raise ValueError(f"num_anchors ({self.num_anchors}) must be divisible by draft CP size "
                             f"({self.draft_context_parallel_size})")
        self._policy = resolve_attention_policy(cfg.to_dict()) if cfg is not None else None
        self.context_shard_alignment = context_shard_alignment(self._policy) if self._policy else 1
        self.context_parallel = None          # set by parallel.context_parallel.attach()
        self._step_counter = 0

    # ------------------------------------------------------------------ policy --
    @property
    def uses_target_distribution(self) -> bool:
        if self._indexer_warmup_kind() is not None:
            return False
        return self.l1_loss_alpha > 0

    @property
    def uses_target_hidden_states(self) -> bool:
        return self.uses_target_distribution or bool(
            self.mtp_conditioning and self.mtp_conditioning["mode"] == "hidden")

    def _prepare_draft_prefix(self, input_ids, last_hidden_states, attention_mask, draft_prefix, *packed_metadata):
        if not self.mtp_conditioning:
            if draft_prefix is not None:
                raise ValueError("Unconditioned Draft does not accept an MTP prefix")
            return None
        if any(v is not None for v in packed_metadata):
            raise ValueError("MTP conditioning does not accept packed or sharded documents")
        if input_ids.shape[0] != 1:
            raise ValueError("MTP conditioning currently requires microbatch size one")
        if draft_prefix is None:
            from aspec_b200.models.dmtp import training_mtp_prefix
            return training_mtp_prefix(self.draft_model, input_ids, last_hidden_states, attention_mask)
        return draft_prefix

    def _block_causal(self, layer: int) -> bool:
        spec = self._policy["draft_block_attention"] if self._policy else "bidirectional"
        if isinstance(spec, list):
            return spec[layer] == "causal"
        return spec.startswith("causal")

    # ----------------------------------------------------------------- anchors --
    def _generator(self, device, anchor_seed: Optional[int]):
        if not self.deterministic_anchor_sampling and anchor_seed is None:
            return None
        seed = anchor_seed if anchor_seed is not None else A.anchor_sampling_seed(
            self.anchor_seed, self._step_counter, 0, 0)
        g = torch.Generator(device=device)
        g.manual_seed(int(seed))
        return g

    def sample_anchors(self, loss_mask, ctx_doc_ids=None, packed_document_lengths=None,
                       attention_mask=None, anchor_seed=None):
        """``(anchors [B, S], keep [B, S])`` by the configured scope, on ``loss_mask``'s device."""
        B, T = loss_mask.shape
        lm = loss_mask
        if ctx_doc_ids is not None:
            # a block must stay inside its anchor's document
            bs = self.block_size
            nxt = torch.full_like(ctx_doc_ids, -2)
            if T > bs:
                nxt[:, : T - bs] = ctx_doc_ids[:, bs:]
            lm = torch.where((ctx_doc_ids >= 0) & (nxt == ctx_doc_ids), lm, torch.zeros_like(lm)) \
                if self.anchor_sampling_scope == "row" else lm
        gen = self._generator(lm.device, anchor_seed)
        if self.anchor_sampling_scope == "sample" and packed_document_lengths is not None:
            return A.sample_document_anchor_positions(
                lm, ctx_doc_ids, tuple(packed_document_lengths), self.num_anchors, self.block_size,
                generator=gen, alignment=max(self.draft_context_parallel_size, 1))
        return A.sample_anchor_positions(T, lm, self.num_anchors, self.block_size, lm.device,
                                         generator=gen, attention_mask=attention_mask)

    @staticmethod
    def _layout(anchors: torch.Tensor, keep: torch.Tensor, seq_len: int, device, compact: bool) -> BlockLayout:
        """Kept blocks in packed order.  With a host-side keep mask the compaction runs on the host and
        one small pinned table is copied asynchronously: no device synchronisation."""
        B, S = anchors.shape
        if not keep.is_cuda and torch.device(device).type == "cuda":
            idx = keep.reshape(-1).nonzero(as_tuple=False).squeeze(-1) if compact else torch.arange(B * S)
            table = torch.stack([idx // S, anchors.cpu().reshape(-1)[idx].long(), idx % S])
            span = None
            if idx.numel():
                flat = table[0] * seq_len + table[1]
                span = (int(flat.min()), int(flat.max()))
            table = table.pin_memory().to(device, non_blocking=True)
            layout = BlockLayout(table[0], table[1], table[2], B, seq_len, S)
            layout.host_span = span
            return layout
        if compact:
            idx = keep.reshape(-1).nonzero(as_tuple=False).squeeze(-1)
        else:
            idx = torch.arange(B * S, device=keep.device)
        idx = idx.to(device)
        return BlockLayout(idx // S, anchors.to(device).reshape(-1)[idx], idx % S, B, seq_len, S)

    # ---------------------------------------------------------------- backbone --
    def _doc_start(self, layout: BlockLayout, ctx_doc_ids, base_position_ids):
        if ctx_doc_ids is None and base_position_ids is None:
            return None
        fa = layout.flat_anchor
        if base_position_ids is not None:
            return layout.anchor - base_position_ids.reshape(-1)[fa].long()
        ids = ctx_doc_ids
        B, T = ids.shape
        pos = torch.arange(T, device=ids.device)[None].expand(B, -1)
        first = torch.ones_like(ids, dtype=torch.bool)
        first[:, 1:] = ids[:, 1:] != ids[:, :-1]
        start = torch.where(first, pos, torch.zeros_like(pos)).cummax(dim=1).values
        return start.reshape(-1)[fa]

    def _draft_backbone(self, input_ids, hidden_states, loss_mask, *, ctx_doc_ids=None,
                        base_position_ids=None, injected_anchors=None, injected_keep_mask=None,
                        anchor_seed=None, packed_document_lengths=None, attention_mask=None,
                        aux: Optional[dict] = None, compact: bool = True, draft_prefix=None):
        B, T = input_ids.shape
        dev = input_ids.device
        bs = self.block_size
        if isinstance(hidden_states, (list, tuple)):
            hidden_states = torch.cat(list(hidden_states), dim=-1)
        if injected_anchors is not None:
            anchors, keep = injected_anchors, injected_keep_mask
            if keep is None:
                raise ValueError("injected anchors need their keep mask")
        else:
            if self.mtp_conditioning:
                # no Target state precedes a document's first token
                loss_mask = loss_mask.clone()
                loss_mask[:, 0] = 0
            anchors, keep = self.sample_anchors(loss_mask, ctx_doc_ids, packed_document_lengths,
                                                attention_mask, anchor_seed)
        self._step_counter += 1
        layout = self._layout(anchors, keep, T, dev, compact)
        n = layout.n
        if not keep.is_cuda and dev.type == "cuda":
            # host-side compaction kept exactly the blocks whose flag is set
            keep_flat = torch.ones(n, dtype=torch.bool, device=dev) if compact else \
                keep.pin_memory().to(dev, non_blocking=True).reshape(-1)
        else:
            keep_flat = keep.to(dev).reshape(-1)[layout.row * layout.n_slots + layout.slot]

        wdtype = self.draft_model.context_proj.weight.dtype
        ctx = self.draft_model.extract_context_feature(hidden_states.reshape(B * T, -1).to(wdtype))
        ctx_pos = (base_position_ids.reshape(-1).long() if base_position_ids is not None
                   else torch.arange(T, device=dev).repeat(B))
        fa = layout.flat_anchor
        j = torch.arange(bs, device=dev)
        noise = torch.full((n, bs), self.draft_model.mask_token_id, dtype=torch.long, device=dev)
        if n:
            noise[:, 0] = torch.where(keep_flat, input_ids.reshape(-1)[fa],
                                      torch.full_like(fa, self.draft_model.mask_token_id))
        embeds = self.draft_model.embed_tokens(noise).reshape(n * bs, -1).to(ctx.dtype)
        if self.mtp_conditioning and n:
            from aspec_b200.models.dmtp import first_candidate_embeddings
            first = first_candidate_embeddings(self.draft_model, input_ids, anchors.to(dev), keep.to(dev), draft_prefix)
            first = first.reshape(-1, first.shape[-1])[layout.row * layout.n_slots + layout.slot]
            embeds = embeds.view(n, bs, -1).clone()
            embeds[:, 1] = first.to(embeds.dtype)
            embeds = embeds.view(n * bs, -1)
        draft_pos = (ctx_pos[fa][:, None] + j[None]).reshape(-1) if n else ctx_pos.new_zeros(0)

        doc_start = self._doc_start(layout, ctx_doc_ids, base_position_ids)
        row_off = layout.row * T
        semantics = self._policy["window_semantics"] if self._policy else "anchor_context"
        tables: List[torch.Tensor] = []
        cache: Dict[tuple, torch.Tensor] = {}
        n_layers = len(self.draft_model.layers)
        for li in range(n_layers):
            window = self._policy["context_windows"][li] if self._policy else None
            causal = self._block_causal(li)
            key = (window, causal)
            if key not in cache:
                cw = window if semantics == "anchor_context" else None
                qw = window if semantics == "query_relative" else None
                ds = (doc_start if doc_start is not None else torch.zeros_like(layout.anchor))
                cache[key] = build_block_intervals(
                    layout.anchor + row_off, keep_flat, ctx_len=B * T, block_size=bs,
                    doc_start=ds + row_off, context_window=cw, query_window=qw, causal=causal)
            tables.append(cache[key])
        cp = self.context_parallel
        if cp is not None and cp.size > 1:
            return self._context_parallel_backbone(cp, hidden_states, B, T, layout, keep_flat, embeds, ctx_pos, draft_pos,
                                                   tables, aux)
        if aux is not None:
            aux["layout"] = layout
            aux["keep"] = keep_flat
            ds_flat = (doc_start if doc_start is not None else torch.zeros_like(layout.anchor)) + row_off
            aux["query_doc_start"] = ds_flat.repeat_interleave(bs)
            aux["query_anchor"] = (layout.anchor + row_off).repeat_interleave(bs)
        hidden = self.draft_model(ctx, embeds, ctx_pos.to(torch.int32), draft_pos.to(torch.int32),
                                  tables, aux)
        return hidden, layout, keep_flat

    def _context_parallel_backbone(self, cp, hidden_states, B, T, layout, keep_flat, embeds, ctx_pos, draft_pos, tables, aux):
        """This rank's share of the backbone: its context rows, its blocks; attention exchanges with the other owners."""
        from aspec_b200.parallel.context_parallel import local_intervals
        allowed = ("full_attention", "sliding_attention", "deepseek_sparse_attention")
        if any(k not in allowed for k in (self._policy or {}).get("layer_types", [])):
            raise NotImplementedError("context parallelism is wired for dense, sliding-window and DSA layers")
        bs, n, total = self.block_size, layout.n, B * T
        s, e = cp.context_bounds(total)
        lo, hi = cp.block_bounds(n)
        wdtype = self.draft_model.context_proj.weight.dtype
        ctx_local = self.draft_model.extract_context_feature(hidden_states.reshape(total, -1)[s:e].to(wdtype))
        q_lo, q_hi = lo * bs, hi * bs
        owners = [cp.block_bounds(n, o) for o in range(cp.size)]
        counts = [(b - a) * bs for a, b in owners]
        per_layer, cache = [], {}
        for t in tables:
            key = id(t)
            if key not in cache:
                cache[key] = {"cp": cp, "counts": counts, "shard": (s, e, total),
                              "tables": [local_intervals(t[a * bs:b * bs], s, e, total, own=(o == cp.rank), query_start=q_lo)
                                         for o, (a, b) in enumerate(owners)]}
            per_layer.append(cache[key])
        hidden = self.draft_model(ctx_local, embeds[q_lo:q_hi], ctx_pos[s:e].to(torch.int32),
                                  draft_pos[q_lo:q_hi].to(torch.int32), per_layer, aux)
        local = BlockLayout(layout.row[lo:hi], layout.anchor[lo:hi], layout.slot[lo:hi], layout.n_rows, layout.seq_len,
                            layout.n_slots)
        return hidden, local, keep_flat[lo:hi]

    # -------------------------------------------------------------- aux losses --
    def _aux_losses(self, aux: dict, weights: torch.Tensor, denominator: torch.Tensor):
        """MoE router / sparse-indexer numerators collected by the layers into ``aux``."""
        total = denominator.new_zeros(())
        comps: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
        cfg = self.draft_model.config
        flat_w = weights.reshape(-1)
        if aux.get("router_logits"):
            if cfg.ffn_type == "ling_moe":
                from aspec_b200.models.draft.ling_moe import ling_router_terms
                num, c = ling_router_terms(aux["router_logits"], flat_w, denominator, cfg.router_z_loss_coef,
                                           cp_group=getattr(self.context_parallel, "group", None))
            else:
                from aspec_b200.models.draft.moe import router_loss_terms
                num, c = router_loss_terms(aux["router_logits"], flat_w, denominator, cfg.num_experts_per_tok,
                                           cp_group=getattr(self.context_parallel, "group", None))
                num = cfg.router_aux_loss_coef * num
            total = total + num
            comps.update(c)
        for kind in ("csa", "qsa", "dsa"):
            losses = aux.get(f"{kind}_losses")
            if losses:
                num = sum((l.to(flat_w.dtype).reshape(-1) * flat_w).sum() for l in losses)
                comps[f"{kind}_indexer_loss"] = (num.detach(), denominator.detach())
                total = total + getattr(cfg, f"{kind}_indexer_loss_coef") * num
        return total, comps

    def _indexer_warmup_kind(self) -> Optional[str]:
        cfg = self.draft_model.config
        for kind in ("csa", "qsa", "dsa"):
            if getattr(cfg, f"{kind}_training_stage", None) == "indexer_warmup":
                return kind
        return None

    def _decay(self, device) -> torch.Tensor:
        k = torch.arange(self.block_size, device=device)
        if self.loss_decay_gamma is not None and self.loss_decay_gamma > 0:
            return torch.exp(-(k - self.prediction_start).clamp_min(0).float() / self.loss_decay_gamma)
        return torch.ones(self.block_size, device=device)

    def _teacher_rows(self, last_hidden_states, flat_index, layout=None):
        """Teacher hidden rows for ``flat_index`` (positions in the flattened ``[B*T]`` context).

        Returns ``(teacher_hidden, t_index)``: the whole context with an index table when that is
        fewer rows than the supervised set (each context row is projected once), else gathered rows.
        """
        flat = last_hidden_states.reshape(-1, last_hidden_states.shape[-1]).to(self.draft_model.context_proj.weight.dtype)
        if self.context_parallel is not None and self.context_parallel.size > 1:
            return self.context_parallel.gather_teacher_rows(flat, flat_index), None
        if layout is not None and layout.host_span is not None:
            # only the context rows between the first anchor and the last block end can be a teacher row
            lo = max(layout.host_span[0] - 1, 0)
            hi = min(layout.host_span[1] + self.block_size + 1, flat.shape[0])
            if hi - lo <= flat_index.numel():
                return flat[lo:hi], (flat_index - lo).to(torch.int32)
        if flat.shape[0] <= flat_index.numel():
            return flat, flat_index.to(torch.int32)
        return flat[flat_index], None

    # ----------------------------------------------------------------- forward --
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
        label = layout.anchor[:, None] + j                                    # [n, bs]
        in_bounds = label < T
        safe = label.clamp(max=T - 1)
        flat_label = layout.row[:, None] * T + safe
        target_ids = input_ids.reshape(-1)[flat_label]
        weight = keep[:, None].float() * in_bounds.float() * (j >= self.prediction_start).float()
        weight = weight * loss_mask.reshape(-1)[flat_label].float()
        binary = weight
        decay = self._decay(dev)[None]

        if self._indexer_warmup_kind() is not None:
            w = binary * (decay if self.loss_objective == "decay" else 1.0)
            den = w.sum()
            num, comps = self._aux_losses(aux, w, den)
            zero = hidden.new_zeros((), dtype=torch.float32)
            pp = hidden.new_zeros(bs, dtype=torch.float32)
            return num / den.clamp_min(1e-6), zero, pp, pp.clone(), pp.clone(), comps, (num, den.detach())

        teacher_hidden = t_index = None
        if self.uses_target_distribution:
            if last_hidden_states is None:
                raise ValueError("DFlash L1 distillation (l1_loss_alpha > 0) requires target last_hidden_states")
            teacher_hidden, t_index = self._teacher_rows(
                last_hidden_states, (layout.row[:, None] * T + (safe - 1).clamp(min=0)).reshape(-1), layout)

        if self.loss_objective == "decay":
            obj_w = binary * decay
        else:
            with torch.no_grad():
                _, ce0, _, _ = head_loss(hidden.detach(), lm_head_weight, target_ids.reshape(-1),
                                         torch.zeros(n * bs, device=dev), a_ce=1.0)
                conf = torch.exp(-ce0.view(n, bs)[:, self.prediction_start:].float())
                dw = torch.ones(n, bs, device=dev)
                if bs > self.prediction_start:
                    dw[:, self.prediction_start:] = dpace_position_weights(conf, self.dpace_alpha)
            obj_w = binary * dw
        num, ce, l1, correct = head_loss(
            hidden, lm_head_weight, target_ids.reshape(-1), obj_w.reshape(-1),
            teacher_hidden=teacher_hidden, t_index=t_index, a_ce=self.ce_loss_alpha,
            a_l1=self.l1_loss_alpha if teacher_hidden is not None else 0.0, chunk_rows=self.num_anchors * bs)
        den = obj_w.sum()
        aux_num, comps = self._aux_losses(aux, obj_w, den)
        num = num + aux_num
        loss = num / den.clamp(min=1e-6)
        with torch.no_grad():
            correct = correct.view(n, bs) * (binary > 0.5)
            accuracy = correct.sum() / binary.sum().clamp(min=1e-6)
            count_pp = binary.sum(0)
            cpp = count_pp.clamp(min=1.0)
            loss_pp = (ce.view(n, bs) * binary).sum(0) / cpp
            acc_pp = correct.sum(0) / cpp
        return loss, accuracy, loss_pp, acc_pp, count_pp, comps, (num, den.detach())
