"""D-MTP: DFlash / DSpark blocks conditioned on a frozen native MTP predictor ("dual anchor").

Block position 0 is the known pending token ``x[a]``; position 1 receives the first candidate ``T1`` - the true
``x[a+1]`` when training (teacher forcing), the MTP's own proposal when drafting.  In ``hidden`` mode the MTP's
post-norm prediction state (row ``a-1``: formed from Target ``h[a-1]`` and token ``x[a]``, predicting ``x[a+1]``) is
fused into that embedding through a zero-initialised residual projection
(reference: aspec/models/dmtp.py:20-181).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn as nn

from aspec_b200.models.draft.mtp import MTPPredictor, causal_intervals, native_key
from aspec_b200.ops.linear import Linear
from aspec_b200.ops.norm import RMSNorm


@dataclass
class MTPPrefix:
    prediction_hidden: Optional[torch.Tensor] = None      # [B, T-1, Dt]: row i predicts x[i+2] after consuming x[i+1]
    first_candidate_ids: Optional[torch.Tensor] = None    # [B, S] one proposal per anchor; None = teacher forced


class MTPAnchorFusion(nn.Module):
    def __init__(self, embedding_size: int, mtp_hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.embedding_norm = RMSNorm(embedding_size, eps=eps)
        self.hidden_norm = RMSNorm(mtp_hidden_size, eps=eps)
        self.proj = Linear(embedding_size + mtp_hidden_size, embedding_size)
        nn.init.zeros_(self.proj.weight)

    def forward(self, embeddings, hidden):
        feats = torch.cat((self.embedding_norm(embeddings), self.hidden_norm(hidden.detach().to(embeddings.dtype))), -1)
        return embeddings + self.proj(feats)


class FrozenMTPFeatures(MTPPredictor):
    """The native predictor body, always frozen and in eval mode; it borrows the draft's Target embedding."""

    def __init__(self, native_config: dict):
        from aspec_b200.config.draft_config import NativeMTPConfig
        super().__init__(NativeMTPConfig(native_config=native_config).native_config)
        self.requires_grad_(False)
        self.eval()

    def train(self, mode: bool = True):
        return super().train(False)

    def initialize_native_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.load_state_dict({n: tensors[native_key(n)] for n in self.state_dict()}, strict=True)
        self.requires_grad_(False)

    @torch.no_grad()
    def validate_native_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for name, actual in self.state_dict().items():
            expected = tensors[native_key(name)]
            if actual.shape != expected.shape or not torch.equal(actual.cpu(), expected.to(actual.dtype).cpu()):
                raise ValueError("Frozen MTP differs from its Target: " + name)

    @torch.no_grad()
    def forward(self, hidden, embeds, positions, intervals):
        return self.predict_embeddings(hidden.detach(), embeds.detach(), positions, intervals).detach()


def training_mtp_prefix(draft, input_ids, last_hidden_states, attention_mask=None) -> MTPPrefix:
    policy = draft.config.mtp_conditioning
    if policy["mode"] == "token":
        return MTPPrefix()
    if last_hidden_states is None or last_hidden_states.shape[:2] != input_ids.shape:
        raise ValueError("MTP hidden conditioning requires aligned post-norm Target final states")
    if input_ids.shape[0] != 1:
        raise ValueError("MTP conditioning currently requires microbatch size one")
    total = input_ids.shape[1]
    length = total
    if attention_mask is not None:
        if attention_mask.shape != input_ids.shape:
            raise ValueError("MTP attention mask must align with input token IDs")
        length = int(attention_mask.sum())
        if not attention_mask[:, :length].bool().all() or attention_mask[:, length:].bool().any():
            raise ValueError("MTP conditioning requires right-padded complete documents")
    width = draft.config.target_hidden_size
    if length < 2:
        return MTPPrefix(last_hidden_states.new_zeros((1, max(total - 1, 0), width)))
    dev = input_ids.device
    pos = torch.arange(length - 1, device=dev, dtype=torch.int32)
    wdtype = draft.mtp_source.fc.weight.dtype
    hidden = draft.mtp_source(last_hidden_states[0, :length - 1].to(wdtype),
                              draft.embed_tokens(input_ids[0, 1:length]).to(wdtype), pos,
                              causal_intervals(torch.zeros(length - 1, dtype=torch.long, device=dev)))
    hidden = torch.nn.functional.pad(hidden, (0, 0, 0, total - length))
    return MTPPrefix(hidden.detach()[None])


def first_candidate_embeddings(draft, input_ids, anchors, keep, prefix: MTPPrefix) -> torch.Tensor:
    """``[B, S, D]`` embedding of ``T1`` per anchor, fused with the MTP state in ``hidden`` mode."""
    if not isinstance(prefix, MTPPrefix):
        raise ValueError("MTP conditioning requires an explicit derived prefix")
    T = input_ids.shape[1]
    if ((anchors < 1) | (anchors + 1 >= T))[keep].any():
        raise ValueError("MTP anchors need a previous Target state and an in-bounds T1")
    if prefix.first_candidate_ids is None:
        ids = input_ids.gather(1, (anchors + 1).clamp(max=T - 1))
    else:
        ids = prefix.first_candidate_ids
        if ids.shape != anchors.shape or ids.dtype != torch.long:
            raise ValueError("MTP proposal IDs must be int64 with the anchor shape")
    ids = torch.where(keep, ids, torch.full_like(ids, draft.mask_token_id))
    first = draft.embed_tokens(ids)
    if draft.config.mtp_conditioning["mode"] == "hidden":
        hidden = prefix.prediction_hidden
        expected = (input_ids.shape[0], T - 1, draft.config.target_hidden_size)
        if hidden is None or tuple(hidden.shape) != expected:
            raise ValueError(f"MTP prediction hidden must have shape {expected}")
        index = (anchors - 1).clamp_min(0).unsqueeze(-1).expand(-1, -1, hidden.shape[-1])
        selected = hidden.gather(1, index)
        selected = torch.where(keep.unsqueeze(-1), selected, torch.zeros_like(selected))
        first = draft.mtp_fusion(first.to(draft.mtp_fusion.proj.weight.dtype), selected)
    elif prefix.prediction_hidden is not None:
        raise ValueError("Token-only conditioning does not consume MTP hidden features")
    return first


def condition_noise_embeddings(draft, embeddings, input_ids, anchors, keep, prefix, block_size):
    """Replace block position 1 of ``embeddings [B, S * block, D]`` with the (fused) ``T1`` embedding."""
    first = first_candidate_embeddings(draft, input_ids, anchors, keep, prefix)
    blocks = embeddings.reshape(input_ids.shape[0], anchors.shape[1], block_size, -1)
    return torch.cat((blocks[:, :, :1], first.unsqueeze(2).to(blocks.dtype), blocks[:, :, 2:]), 2).flatten(1, 2)


@torch.no_grad()
def frozen_mtp_predictions(mtp, input_ids, final_hidden_states):
    """Causal single-document predictor pass: output row ``a-1`` predicts the unverified ``x[a+1]``."""
    if mtp.training or any(p.requires_grad for p in mtp.parameters()):
        raise ValueError("The native MTP feature producer must be frozen and in eval mode")
    if (input_ids.ndim != 2 or input_ids.shape[0] != 1 or input_ids.shape[1] < 2
            or final_hidden_states.shape[:2] != input_ids.shape):
        raise ValueError("MTP feature extraction requires one complete unpadded document")
    n = input_ids.shape[1] - 1
    dev = input_ids.device
    pos = torch.arange(n, device=dev, dtype=torch.int32)
    out = mtp.predict(final_hidden_states[0, :-1].detach(), input_ids[0, 1:], pos,
                      causal_intervals(torch.zeros(n, dtype=torch.long, device=dev)))
    return out.detach()[None]
