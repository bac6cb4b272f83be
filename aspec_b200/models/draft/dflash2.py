"""DFlash2 draft: DFlash decoder layers wrapped in per-block grouped causal convolutions with input-dependent
kernels, plus a low-rank pairwise candidate selector over the unary top-k
(reference: aspec/models/draft/dflash2.py:312-514).

* ``DFlashGroupedConv``: a static ``base_kernel [2, K, D]`` (initialised to identity) plus a dynamic kernel
  ``kernel_projection(x) -> [2, K, D/group]`` (zero-initialised); side 0 is applied before the sub-layer
  (``prepare``), side 1 after it (``finish``) with the kernel computed from the pre-sub-layer input.  The
  convolution is causal inside each ``block_size`` block and never crosses blocks.
* ``CandidateSelector``: ``score(c) = unary(c) + <P[prev] * W h, S[c]>`` over the top-k unary candidates; in
  training the true successor replaces the weakest candidate when it is missing.
"""
from __future__ import annotations

import json
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.config.draft_config import DFlash2Config
from aspec_b200.models.draft.dflash import DFlashDecoderLayer, DFlashDraftModel
from aspec_b200.ops.linear import Linear

_NESTED_FIELDS = ("attention_mode", "block_size", "conv_group_size", "conv_kernel_size", "final_logit_softcapping",
                  "input_embedding_scale", "mask_token_id", "output_multiplier", "selector_rank", "selector_top_k",
                  "target_layer_ids")
_SERVING_PREFIXES = (("context_proj.", "fc."), ("context_norm.", "hidden_norm."), ("final_norm.", "norm."))


def dflash2_config_for_serving(raw: dict, *, export_for_vllm: bool = False) -> dict:
    """Serving engines read the DFlash2 extras from a nested ``dflash_config`` under a ``qwen3`` model type."""
    cfg = json.loads(json.dumps(raw))
    nested = dict(cfg.get("dflash_config") or {})
    for key in _NESTED_FIELDS:
        if key in cfg:
            nested.setdefault(key, cfg[key])
        cfg.pop(key, None)
    cfg["dflash_config"] = nested
    n_target = cfg.pop("target_num_hidden_layers", None)
    if n_target is not None:
        cfg["num_target_layers"] = n_target
    if not export_for_vllm and float(nested.get("input_embedding_scale", 1.0)) != 1.0:
        raise ValueError("SGLang DFlash2 export requires input_embedding_scale=1.0")
    cfg.pop("target_hidden_size", None)
    cfg["model_type"] = "qwen3"
    if "sliding_attention" in (cfg.get("layer_types") or []):
        cfg["use_sliding_window"] = True
    return cfg


def dflash2_state_dict_for_serving(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for key, value in state.items():
        if key == "embed_tokens.weight":
            continue
        for old, new in _SERVING_PREFIXES:
            if key.startswith(old):
                key = new + key[len(old):]
                break
        out[key] = value
    return out


class DFlashGroupedConv(nn.Module):
    def __init__(self, hidden_size: int, block_size: int, kernel_size: int, group_size: int):
        super().__init__()
        if hidden_size % group_size:
            raise ValueError(f"group_size={group_size} must divide hidden_size={hidden_size}")
        self.block_size, self.kernel_size, self.group_size = int(block_size), int(kernel_size), int(group_size)
        self.num_groups = hidden_size // self.group_size
        base = torch.zeros(2, self.kernel_size, hidden_size)
        base[:, 0] = 1.0
        self.base_kernel = nn.Parameter(base)
        self.kernel_projection = Linear(hidden_size, 2 * self.kernel_size * self.num_groups)
        nn.init.zeros_(self.kernel_projection.weight)

    def _convolve(self, x: torch.Tensor, dynamic: torch.Tensor, side: int) -> torch.Tensor:
        """``x [N, D]`` (N a multiple of the block), ``dynamic [N, K, groups]``."""
        n, D = x.shape
        if n % self.block_size:
            raise ValueError(f"draft length {n} must be divisible by block_size={self.block_size}")
        blocks = x.view(-1, self.block_size, self.num_groups, self.group_size)
        dyn = dynamic.reshape(-1, self.block_size, self.kernel_size, self.num_groups)
        out = torch.zeros_like(blocks)
        for off in range(min(self.kernel_size, self.block_size)):
            vals = blocks if off == 0 else F.pad(blocks[:, :-off], (0, 0, 0, 0, off, 0))
            base = self.base_kernel[side, off].to(x.dtype).view(1, 1, self.num_groups, self.group_size)
            out = out + (base + dyn[:, :, off, :, None].to(x.dtype)) * vals
        return out.reshape(n, D)

    def prepare(self, x: torch.Tensor):
        dyn = self.kernel_projection(x).view(x.shape[0], 2, self.kernel_size, self.num_groups)
        return self._convolve(x, dyn[:, 0], 0), dyn[:, 1]

    def finish(self, x: torch.Tensor, dynamic: torch.Tensor) -> torch.Tensor:
        return self._convolve(x, dynamic, 1)


class CandidateSelector(nn.Module):
    def __init__(self, hidden_size: int, vocab_size: int, rank: int, top_k: int):
        super().__init__()
        if not 2 <= top_k <= vocab_size:
            raise ValueError(f"top_k must be in [2, {vocab_size}], got {top_k}")
        self.top_k = int(top_k)
        self.predecessor_codebook = nn.Parameter(torch.empty(vocab_size, rank))
        self.successor_codebook = nn.Parameter(torch.empty(vocab_size, rank))
        self.hidden_projection = Linear(hidden_size, rank)
        nn.init.normal_(self.predecessor_codebook, std=0.02)
        nn.init.normal_(self.successor_codebook, std=0.02)

    def score_candidates(self, hidden, logits, predecessor_ids, *, training_successor_ids=None):
        unary, cand = torch.topk(logits, self.top_k, dim=-1, sorted=False)
        if training_successor_ids is not None:
            truth = training_successor_ids.unsqueeze(-1)
            missing = ~(cand == truth).any(-1, keepdim=True)
            slot = unary.argmin(-1, keepdim=True)
            cand = cand.scatter(-1, slot, torch.where(missing, truth, cand.gather(-1, slot)))
            unary = unary.scatter(-1, slot, torch.where(missing, logits.gather(-1, truth), unary.gather(-1, slot)))
        h = self.hidden_projection(hidden).float()
        pred = self.predecessor_codebook[predecessor_ids].float() * h
        succ = self.successor_codebook[cand].float()
        return unary + torch.einsum("...r,...kr->...k", pred, succ), cand


class DFlash2DecoderLayer(DFlashDecoderLayer):
    def __init__(self, config, layer_idx: int = 0):
        super().__init__(config, layer_idx)
        args = (config.hidden_size, config.block_size, config.conv_kernel_size, config.conv_group_size)
        self.attention_conv = DFlashGroupedConv(*args)
        self.mlp_conv = DFlashGroupedConv(*args)

    def forward(self, x, ctx, q_pos, kv_pos, intervals, aux=None):
        h, kern = self.attention_conv.prepare(self.input_layernorm(x))
        h = self.self_attn(h, ctx, q_pos, kv_pos, intervals, aux=aux)
        x = x + self.attention_conv.finish(h, kern)
        h, kern = self.mlp_conv.prepare(self.post_attention_layernorm(x))
        h = self.mlp(h, aux=aux) if getattr(self.mlp, "wants_aux", False) else self.mlp(h)
        return x + self.mlp_conv.finish(h, kern)


class DFlash2DraftModel(DFlashDraftModel):
    config_class = DFlash2Config
    decoder_layer_class = DFlash2DecoderLayer

    def __init__(self, config):
        super().__init__(config)
        self.candidate_selector = CandidateSelector(config.hidden_size, config.vocab_size, config.selector_rank,
                                                    config.selector_top_k)

    def config_for_serving(self) -> dict:
        return dflash2_config_for_serving(self.config.to_dict())

    def state_dict_for_serving(self, state: Optional[dict] = None) -> dict:
        return dflash2_state_dict_for_serving(self.state_dict() if state is None else state)

    def forward(self, context_feature, draft_embeds, context_positions, draft_positions, intervals, aux=None):
        return super().forward(context_feature, draft_embeds * self.config.input_embedding_scale,
                               context_positions, draft_positions, intervals, aux)
