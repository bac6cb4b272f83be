"""EAGLE4 draft: the EAGLE3 recurrent layer with an optional embed/hidden fusion projection ahead of attention,
an optional post-MLP norm on the recurrent state, sliding-window attention, an optional MoE feed-forward, and a
low-rank candidate-retrieval head trained in a second stage (reference: aspec/models/draft/eagle4.py:40-198).

Stages: ``draft`` trains everything but the candidate head; ``candidate_head`` freezes the draft body (kept in eval
mode) and trains ``efficient_lm_head_down_proj`` / ``efficient_lm_head`` to reproduce the frozen draft's top-k
distribution, starting from a randomised truncated SVD of the exact head.
"""
from __future__ import annotations

import torch

from aspec_b200.config.draft_attention import resolve_attention_policy
from aspec_b200.config.draft_config import Eagle4Config
from aspec_b200.config.eagle4 import eagle4_policy
from aspec_b200.models.draft.eagle4_moe import Eagle4MoE, split_latent_experts, stack_latent_experts
from aspec_b200.models.draft.keymap import to_export_keys, to_internal_keys
from aspec_b200.models.draft.llama3_eagle import EagleAttention, EagleDecoderLayer, LlamaForCausalLMEagle3
from aspec_b200.ops.linear import Linear
from aspec_b200.ops.norm import RMSNorm

_CANDIDATE_PREFIXES = ("efficient_lm_head.", "efficient_lm_head_down_proj.")


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
    def candidate_stage(self) -> bool:
        return self.eagle4_policy["stage"] == "candidate_head"

    @property
    def preserve_loaded_embedding(self) -> bool:
        return self.candidate_stage

    def configure_training_stage(self) -> None:
        for name, p in self.named_parameters():
            cand = name.startswith(_CANDIDATE_PREFIXES)
            p.requires_grad_(cand if self.candidate_stage else not cand)
        self.embed_tokens.weight.requires_grad_(False)
        if self.norm_output and hasattr(self.midlayer, "post_mlp_layernorm"):
            self.midlayer.post_mlp_layernorm.requires_grad_(False)
        self.train(self.training)

    def train(self, mode: bool = True):
        super().train(mode)
        if hasattr(self, "eagle4_policy") and self.candidate_stage:
            for name, module in self.named_children():
                if name not in ("efficient_lm_head", "efficient_lm_head_down_proj"):
                    module.eval()
        return self

    def validate_target_binding(self, target_embedding: torch.Tensor) -> None:
        if self.candidate_stage:
            actual = self.embed_tokens.weight.detach()
            if actual.shape != target_embedding.shape or not torch.equal(actual.cpu(), target_embedding.to(actual.dtype).cpu()):
                raise ValueError("Candidate training requires the pretrained Draft's same frozen Target embedding")

    @torch.no_grad()
    def initialize_candidate_head(self, *, device=None) -> None:
        if int(self.candidate_head_steps) != 0:
            raise ValueError("Refusing to overwrite a trained candidate head with SVD")
        weight = self.lm_head.weight.detach().to(device=device, dtype=torch.float32)
        rank = self.eagle4_policy["rank"]
        u, s, v = torch.svd_lowrank(weight, q=min(rank + 16, *weight.shape), niter=2)
        self.efficient_lm_head_down_proj.weight.copy_(v[:, :rank].T)
        self.efficient_lm_head.weight.copy_(u[:, :rank] * s[:rank])

    def candidate_scores(self, hidden):
        return self.efficient_lm_head(self.efficient_lm_head_down_proj(hidden))

    @torch.no_grad()
    def score_candidates(self, hidden):
        """Exact draft logits on the retrieved shortlist (evaluation helper, not a serving path)."""
        ids = self.candidate_scores(hidden).topk(self.eagle4_policy["num_candidates"], -1).indices
        return ids, torch.matmul(self.lm_head.weight[ids], hidden.unsqueeze(-1)).squeeze(-1)

    def commit_router_load(self) -> None:
        mlp = self.midlayer.mlp
        if self.training and not self.candidate_stage and isinstance(mlp, Eagle4MoE) and mlp.last_load is not None:
            mlp.gate.load.add_(mlp.last_load)

    def state_dict_from_serving(self, tensors: dict) -> dict:
        return to_internal_keys(stack_latent_experts(tensors), self.state_dict().keys())

    def state_dict_for_serving(self) -> dict:
        return split_latent_experts(to_export_keys(self.state_dict()))
