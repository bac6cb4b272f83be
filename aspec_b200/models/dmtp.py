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


def read_native_mtp_tensors(checkpoint_dir: str) -> Dict[str, torch.Tensor]:
    """The ``mtp.*`` tensors of a Target checkpoint directory (safetensors, single file or sharded with
    ``model.safetensors.index.json``; also the output of ``stitch-mtp``).  Only the shards that hold them are opened.
    (reference: native predictor initialisation, aspec/training/mtp_trainer.py:24-61)"""
    import json
    import os
    from safetensors import safe_open
    index = os.path.join(checkpoint_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        weight_map = json.load(open(index))["weight_map"]
        shards = sorted({f for k, f in weight_map.items() if k.startswith("mtp.")})
    else:
        shards = sorted(f for f in os.listdir(checkpoint_dir) if f.endswith(".safetensors"))
    out: Dict[str, torch.Tensor] = {}
    for shard in shards:
        with safe_open(os.path.join(checkpoint_dir, shard), framework="pt") as f:
            for key in f.keys():
                if key.startswith("mtp."):
                    out[key] = f.get_tensor(key)
    return out


def _document_length(input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor]) -> int:
    """Tokens of the (single, right-padded) document in the row."""
    total = input_ids.shape[1]
    if attention_mask is None:
        return total
    if attention_mask.shape != input_ids.shape:
        raise ValueError(f"attention mask {tuple(attention_mask.shape)} does not cover the ids {tuple(input_ids.shape)}")
    live = attention_mask[0].bool()
    n = int(live.sum())
    if not bool(live[:n].all()) or bool(live[n:].any()):
        raise ValueError("the MTP prefix needs one contiguous document followed by padding only")
    return n


def training_mtp_prefix(draft, input_ids, last_hidden_states, attention_mask=None) -> MTPPrefix:
    """What the training wrapper hands to the block model: nothing in ``token`` mode (the first candidate is teacher
    forced), the frozen predictor's post-norm states ``[1, T-1, Dt]`` in ``hidden`` mode."""
    if draft.config.mtp_conditioning["mode"] != "hidden":
        return MTPPrefix()
    rows, total = input_ids.shape
    if rows != 1:
        raise ValueError("MTP-conditioned training takes one row per micro-batch")
    if last_hidden_states is None or tuple(last_hidden_states.shape[:2]) != (rows, total):
        raise ValueError("hidden-mode conditioning needs the Target's final (post-norm) state of every token")
    n = _document_length(input_ids, attention_mask)
    width = draft.config.target_hidden_size
    if n < 2:                                              # nothing to predict from
        return MTPPrefix(last_hidden_states.new_zeros(1, max(total - 1, 0), width))
    source = draft.mtp_source
    dtype = source.fc.weight.dtype
    steps = n - 1                                          # row i: Target state of token i and token i+1 -> token i+2
    device = input_ids.device
    states = source(last_hidden_states[0, :steps].to(dtype), draft.embed_tokens(input_ids[0, 1:n]).to(dtype),
                    torch.arange(steps, device=device, dtype=torch.int32),
                    causal_intervals(torch.zeros(steps, dtype=torch.long, device=device)))
    padded = states.new_zeros(total - 1, states.shape[-1])
    padded[:steps] = states
    return MTPPrefix(padded.detach().unsqueeze(0))


def first_candidate_embeddings(draft, input_ids, anchors, keep, prefix: MTPPrefix) -> torch.Tensor:
    """``[B, S, D]``: the embedding of every anchor's first candidate ``T1`` (fused with the predictor's state in
    ``hidden`` mode).  ``T1`` is ``x[a+1]`` when ``prefix.first_candidate_ids`` is ``None`` (training), else the given
    proposals (drafting); dropped anchors get the mask token."""
    if not isinstance(prefix, MTPPrefix):
        raise ValueError("pass the MTPPrefix derived for this row (training_mtp_prefix or a proposal-time prefix)")
    mode = draft.config.mtp_conditioning["mode"]
    batch, length = input_ids.shape
    live = anchors[keep]
    if live.numel() and (int(live.min()) < 1 or int(live.max()) + 1 >= length):
        raise ValueError("every kept anchor needs a token before it (the predictor's input) and one after it (T1)")
    proposals = prefix.first_candidate_ids
    if proposals is None:
        proposals = torch.gather(input_ids, 1, torch.clamp(anchors + 1, max=length - 1))
    elif proposals.dtype != torch.long or proposals.shape != anchors.shape:
        raise ValueError("first_candidate_ids must be an int64 tensor shaped like the anchors")
    proposals = proposals.masked_fill(~keep, draft.mask_token_id)
    embedded = draft.embed_tokens(proposals)
    states = prefix.prediction_hidden
    if mode != "hidden":
        if states is not None:
            raise ValueError("token-mode conditioning takes no predictor states")
        return embedded
    want = (batch, length - 1, draft.config.target_hidden_size)
    if states is None or tuple(states.shape) != want:
        raise ValueError(f"hidden-mode conditioning expects predictor states of shape {want}")
    rows = torch.clamp(anchors - 1, min=0)                                  # state a-1 predicts x[a+1]
    picked = torch.gather(states, 1, rows[..., None].expand(*rows.shape, states.shape[-1]))
    picked = picked * keep[..., None].to(picked.dtype)
    fusion = draft.mtp_fusion
    return fusion(embedded.to(fusion.proj.weight.dtype), picked)


def condition_noise_embeddings(draft, embeddings, input_ids, anchors, keep, prefix, block_size):
    """Put the (fused) ``T1`` embedding into slot 1 of every block of ``embeddings [B, S * block, D]``."""
    first = first_candidate_embeddings(draft, input_ids, anchors, keep, prefix)
    blocks = embeddings.view(input_ids.shape[0], anchors.shape[1], block_size, embeddings.shape[-1]).clone()
    blocks[:, :, 1] = first.to(blocks.dtype)
    return blocks.view(input_ids.shape[0], -1, embeddings.shape[-1])


@torch.no_grad()
def frozen_mtp_predictions(mtp, input_ids, final_hidden_states):
    """Predictor states ``[1, T-1, Dt]`` of one whole document (proposal time): row ``a-1`` is the state that predicts
    ``x[a+1]``.  The predictor must be frozen and in eval mode."""
    trainable = [n for n, p in mtp.named_parameters() if p.requires_grad]
    if mtp.training or trainable:
        raise ValueError("the native MTP predictor is a frozen feature producer: call .eval() and freeze it first")
    one_document = input_ids.ndim == 2 and input_ids.shape[0] == 1 and input_ids.shape[1] >= 2
    if not one_document or tuple(final_hidden_states.shape[:2]) != tuple(input_ids.shape):
        raise ValueError("expected one unpadded document of at least two tokens with a final state per token")
    steps = input_ids.shape[1] - 1
    device = input_ids.device
    states = mtp.predict(final_hidden_states[0, :steps].detach(), input_ids[0, 1:],
                         torch.arange(steps, device=device, dtype=torch.int32),
                         causal_intervals(torch.zeros(steps, dtype=torch.long, device=device)))
    return states.detach().unsqueeze(0)
