"""Shared pieces of the EAGLE-family drafts: vocabulary buffers, low-rank head, weight loading
(reference: aspec/models/draft/base.py:98-375)."""
from __future__ import annotations

import json
import os

import torch
import torch.nn as nn

from aspec_b200.ops.linear import Linear


class LowRankHead(nn.Module):
    """``up(down(h))``: a rank-``r`` stand-in for a ``[V, D]`` head (EAGLE4 candidate retrieval)."""

    def __init__(self, hidden_size: int, vocab_size: int, rank: int):
        super().__init__()
        self.down = Linear(hidden_size, rank)
        self.up = Linear(rank, vocab_size)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.up(self.down(h))

    @torch.no_grad()
    def init_from_dense(self, weight: torch.Tensor, oversample: int = 8, seed: int = 0) -> None:
        """Randomised truncated SVD of a dense head ``W [V, D]``: ``W ~= U S Vh`` -> up = U S, down = Vh."""
        r = self.down.weight.shape[0]
        g = torch.Generator(device="cpu").manual_seed(seed)
        W = weight.float().cpu()
        omega = torch.randn(W.shape[1], min(r + oversample, W.shape[1]), generator=g)
        Q, _ = torch.linalg.qr(W @ omega)
        U_small, S, Vh = torch.linalg.svd(Q.t() @ W, full_matrices=False)
        U = Q @ U_small
        self.up.weight.copy_((U[:, :r] * S[:r]).to(self.up.weight))
        self.down.weight.copy_(Vh[:r].to(self.down.weight))


def load_tensor_from_pretrained(model_path: str, key: str) -> torch.Tensor:
    """Reads one tensor from a HF-style checkpoint directory (safetensors, sharded or not)."""
    from safetensors import safe_open
    index = os.path.join(model_path, "model.safetensors.index.json")
    if os.path.isfile(index):
        fname = json.load(open(index))["weight_map"][key]
    else:
        fname = "model.safetensors"
    with safe_open(os.path.join(model_path, fname), framework="pt") as f:
        return f.get_tensor(key)


class Eagle3DraftModel(nn.Module):
    """Base of drafts that own an output head over a (possibly pruned) draft vocabulary."""

    def init_vocab_buffers(self, vocab_size: int, draft_vocab_size: int) -> None:
        self.target_vocab_size, self.draft_vocab_size = int(vocab_size), int(draft_vocab_size)
        self.register_buffer("t2d", torch.ones(vocab_size, dtype=torch.bool) if draft_vocab_size == vocab_size
                             else torch.zeros(vocab_size, dtype=torch.bool))
        self.register_buffer("d2t", torch.zeros(draft_vocab_size, dtype=torch.int64))

    def set_vocab_buffers(self, d2t: torch.Tensor, t2d: torch.Tensor) -> None:
        from aspec_b200.models.vocab import validate_vocab_mapping
        validate_vocab_mapping(d2t, t2d, self.draft_vocab_size, self.target_vocab_size)
        self.d2t.copy_(d2t)
        self.t2d.copy_(t2d)

    @property
    def vocab_pruned(self) -> bool:
        return self.draft_vocab_size != self.target_vocab_size

    def load_embedding(self, source, embedding_key: str = "model.embed_tokens.weight") -> None:
        weight = source if torch.is_tensor(source) else load_tensor_from_pretrained(source, embedding_key)
        with torch.no_grad():
            self.embed_tokens.weight.copy_(weight.to(self.embed_tokens.weight))
        self.embed_tokens.weight.requires_grad_(False)

    def load_lm_head(self, source, lm_head_key: str = "lm_head.weight") -> None:
        weight = source if torch.is_tensor(source) else load_tensor_from_pretrained(source, lm_head_key)
        if self.vocab_pruned:
            weight = weight[self.t2d.to(weight.device)]
        with torch.no_grad():
            self.lm_head.weight.copy_(weight.to(self.lm_head.weight))
