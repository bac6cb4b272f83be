"""EAGLE4 draft: the EAGLE3 recurrent layer with an optional embed/hidden fusion projection ahead of attention,
an optional post-MLP norm on the recurrent state, sliding-window attention, an optional MoE feed-forward, and a
low-rank candidate-retrieval head trained in a second stage (reference: aspec/models/draft/eagle4.py:40-198).

Stages: ``draft`` trains everything but the candidate head; ``candidate_head`` freezes the draft body (kept in eval
mode) and trains ``efficient_lm_head_down_proj`` / ``efficient_lm_head`` to reproduce the frozen draft's top-k
distribution, starting from the rank-r truncation of the exact head (``models/draft/candidate_head.py``).
"""
from __future__ import annotations

import torch

from aspec_b200.config.draft_attention import resolve_attention_policy
from aspec_b200.config.draft_config import Eagle4Config
from aspec_b200.config.eagle4 import eagle4_policy
from aspec_b200.models.draft.candidate_head import CANDIDATE_MODULES, low_rank_factors, shortlist_logits, stage_trains
from aspec_b200.models.draft.eagle4_moe import Eagle4MoE, split_latent_experts, stack_latent_experts
from aspec_b200.models.draft.keymap import to_export_keys, to_internal_keys
from aspec_b200.models.draft.llama3_eagle import EagleAttention, EagleDecoderLayer, LlamaForCausalLMEagle3
from aspec_b200.ops.linear import Linear
from aspec_b200.ops.norm import RMSNorm


class Eagle4DecoderLayer(EagleDecoderLayer):
    def __init__(self, config):
        super().__init__(config)
        D = config.hidden_size
        fused = bool(getattr(config, "attn_norm", False))
        window = resolve_attention_policy(config.to_dict())["context_windows"][0]
        self.self_attn = EagleAttention(config, input_width=D if fused else 2 * D,
                                        use_rope=bool(getattr(config, "use_rope", True)), window=window)
        if getattr(config, "enable_moe", False):
            self.mlp = Eagle4MoE(config)
        if fused:
            self.eh_proj = Linear(2 * D, D)
            self.pre_attention_layernorm = RMSNorm(D, eps=config.rms_norm_eps)
        if getattr(config, "enable_post_mlp_norm", False):
            self.post_mlp_layernorm = RMSNorm(D, eps=config.rms_norm_eps)

    def attention_input(self, embeds, hidden):
        x, residual = super().attention_input(embeds, hidden)
        if hasattr(self, "eh_proj"):
            residual = self.eh_proj(x)
            x = self.pre_attention_layernorm(residual)
        return x, residual


class Eagle4DraftModel(LlamaForCausalLMEagle3):
    config_class = Eagle4Config
    decoder_layer_class = Eagle4DecoderLayer

    def __init__(self, config):
        super().__init__(config)
        self.eagle4_policy = eagle4_policy(config.to_dict())
        self.sliding_window = self.midlayer.self_attn.window
        rank = self.eagle4_policy["rank"]
        self.efficient_lm_head_down_proj = Linear(config.hidden_size, rank)
        self.efficient_lm_head = Linear(rank, config.vocab_size)
        self.register_buffer("candidate_head_steps", torch.zeros((), dtype=torch.long))
        self._valid_rows = None

    # -- recurrence hooks -----------------------------------------------------------------------
    def next_depth_hidden(self, hidden):
        if self.norm_output:
            return self.norm(hidden)
        norm = getattr(self.midlayer, "post_mlp_layernorm", None)
        return hidden if norm is None else norm(hidden)

    def _mlp(self, layer, x, depth):
        mlp = layer.mlp
        if isinstance(mlp, Eagle4MoE):
            mlp.query_mask = self._valid_rows(depth) if callable(self._valid_rows) else None
            try:
                return mlp(x)
            finally:
                mlp.query_mask = None
        return mlp(x)

    def set_valid_rows(self, fn) -> None:
        """``fn(depth) -> bool [T]``: rows whose depth-shifted query still lies inside its document."""
        self._valid_rows = fn

    # -- stages ---------------------------------------------------------------------------------------
    @property
    def stage(self) -> str:
        return self.eagle4_policy["stage"]

    @property
    def candidate_stage(self) -> bool:
        return self.stage == "candidate_head"

    @property
    def preserve_loaded_embedding(self) -> bool:
        # the candidate stage distils a finished Draft: its embedding must stay the one it was trained with
        return self.candidate_stage

    def _frozen_body(self):
        """Sub-modules that stay in inference mode while only the candidate head trains."""
        return [m for name, m in self.named_children() if name not in CANDIDATE_MODULES]

    def configure_training_stage(self) -> None:
        """Mark what the configured stage updates; the embedding is the Target's and never trains, and a post-MLP norm
        that ``norm_output`` bypasses would be a trainable leaf nothing reaches."""
        stage = self.stage
        for name, param in self.named_parameters():
            param.requires_grad_(stage_trains(name, stage))
        self.embed_tokens.weight.requires_grad_(False)
        bypassed = getattr(self.midlayer, "post_mlp_layernorm", None) if self.norm_output else None
        if bypassed is not None:
            bypassed.requires_grad_(False)
        self.train(self.training)

    def train(self, mode: bool = True):
        super().train(mode)
        # called by nn.Module.__init__ paths before the policy exists
        if getattr(self, "eagle4_policy", None) is not None and self.candidate_stage:
            for module in self._frozen_body():
                module.train(False)
        return self

    def validate_target_binding(self, target_embedding: torch.Tensor) -> None:
        if not self.candidate_stage:
            return
        mine = self.embed_tokens.weight.detach().cpu()
        theirs = target_embedding.detach().to(mine.dtype).cpu()
        if mine.shape != theirs.shape or not torch.equal(mine, theirs):
            raise ValueError("the candidate stage distils a pretrained Draft and needs the Target embedding that Draft was "
                             "trained with; the loaded embedding differs")

    @torch.no_grad()
    def initialize_candidate_head(self, *, device=None) -> None:
        """Start the two projections from the rank-r truncation of the exact head (once: never over trained weights)."""
        if int(self.candidate_head_steps) > 0:
            raise ValueError(f"the candidate head has already taken {int(self.candidate_head_steps)} update(s); "
                             "re-initialising it from the exact head would discard them")
        down, up = low_rank_factors(self.lm_head.weight.detach().to(device=device), self.eagle4_policy["rank"])
        self.efficient_lm_head_down_proj.weight.copy_(down.to(self.efficient_lm_head_down_proj.weight))
        self.efficient_lm_head.weight.copy_(up.to(self.efficient_lm_head.weight))

    def candidate_scores(self, hidden):
        latent = self.efficient_lm_head_down_proj(hidden)
        return self.efficient_lm_head(latent)

    @torch.no_grad()
    def score_candidates(self, hidden):
        """``(ids, exact logits)`` of the retrieved shortlist (an evaluation helper, not the serving path)."""
        k = self.eagle4_policy["num_candidates"]
        ids = torch.topk(self.candidate_scores(hidden), k, dim=-1).indices
        return ids, shortlist_logits(self.lm_head.weight, hidden, ids)

    def commit_router_load(self) -> None:
        """Fold the last forward's expert load into the router's running count (draft stage, training mode only)."""
        if not self.training or self.candidate_stage:
            return
        mlp = self.midlayer.mlp
        load = getattr(mlp, "last_load", None) if isinstance(mlp, Eagle4MoE) else None
        if load is not None:
            mlp.gate.load += load

    # -- serving layout: per-expert latent tensors, exported key names ----------------------------------
    def state_dict_from_serving(self, tensors: dict) -> dict:
        stacked = stack_latent_experts(tensors)
        return to_internal_keys(stacked, self.state_dict().keys())

    def state_dict_for_serving(self) -> dict:
        exported = to_export_keys(self.state_dict())
        return split_latent_experts(exported)
