"""Native multi-token-prediction (MTP) draft of a Qwen3.5-style Target: the Target's own MTP layer
(``pre_fc_norm_embedding`` / ``pre_fc_norm_hidden`` -> ``fc(2D -> D)`` -> one gated full-attention decoder layer ->
``norm``), with the Target's embedding and LM head bound and frozen
(reference: aspec/models/draft/mtp.py:33-202).

The decoder layer is written here rather than borrowed from a model library: zero-centred RMSNorm
(``x * rsqrt(mean x^2 + eps) * (1 + w)``), ``q_proj`` producing query and output gate side by side per head,
per-head q/k norm, partial rotate-half RoPE (text positions: the three multimodal position streams coincide),
causal same-document attention, ``sigmoid(gate)`` on the attention output, SwiGLU MLP.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn

from aspec_b200.config.draft_config import NativeMTPConfig
from aspec_b200.models.draft.base import Eagle3DraftModel
from aspec_b200.models.draft.dflash import DFlashMLP
from aspec_b200.models.draft.sparse_common import rotary
from aspec_b200.ops.attention import interval_attention
from aspec_b200.ops.linear import Linear


class ZeroCenteredRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.zeros(dim))

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * (1.0 + self.weight.float())).type_as(x)


class GatedAttention(nn.Module):
    def __init__(self, native: dict):
        super().__init__()
        D, self.num_heads, self.num_kv_heads = native["hidden_size"], native["num_attention_heads"], native["num_key_value_heads"]
        d = self.head_dim = native["head_dim"]
        bias = bool(native.get("attention_bias", False))
        if bias:
            raise NotImplementedError("attention_bias is not part of the shared-embedding MTP recipe")
        self.q_proj = Linear(D, self.num_heads * d * 2)
        self.k_proj = Linear(D, self.num_kv_heads * d)
        self.v_proj = Linear(D, self.num_kv_heads * d)
        self.o_proj = Linear(self.num_heads * d, D)
        self.q_norm = ZeroCenteredRMSNorm(d, native["rms_norm_eps"])
        self.k_norm = ZeroCenteredRMSNorm(d, native["rms_norm_eps"])
        rope = dict(native.get("rope_parameters") or {})
        self.rope_theta = float(rope.get("rope_theta", native.get("rope_theta", 10000.0)))
        factor = float(rope.get("partial_rotary_factor", native.get("partial_rotary_factor", 1.0)))
        self.rotary_dim = int(d * factor) // 2 * 2
        self.scale = d ** -0.5

    def forward(self, x, positions, intervals):
        T, d = x.shape[0], self.head_dim
        qg = self.q_proj(x).view(T, self.num_heads, 2 * d)
        q, gate = qg[..., :d], qg[..., d:].reshape(T, -1)
        q = rotary(self.q_norm(q), positions, self.rotary_dim, self.rope_theta)
        k = rotary(self.k_norm(self.k_proj(x).view(T, self.num_kv_heads, d)), positions, self.rotary_dim, self.rope_theta)
        v = self.v_proj(x).view(T, self.num_kv_heads, d)
        o, _ = interval_attention(q.contiguous(), k.contiguous(), v.contiguous(), intervals, self.scale)
        return self.o_proj(o.reshape(T, -1) * torch.sigmoid(gate))


class MTPDecoderLayer(nn.Module):
    def __init__(self, native: dict):
        super().__init__()
        D, eps = native["hidden_size"], native["rms_norm_eps"]
        self.self_attn = GatedAttention(native)
        self.mlp = DFlashMLP(D, native["intermediate_size"])
        self.input_layernorm = ZeroCenteredRMSNorm(D, eps)
        self.post_attention_layernorm = ZeroCenteredRMSNorm(D, eps)

    def forward(self, x, positions, intervals):
        x = x + self.self_attn(self.input_layernorm(x), positions, intervals)
        return x + self.mlp(self.post_attention_layernorm(x))


class MTPPredictor(nn.Module):
    """The predictor body without embedding or head: shared by the trainable draft and the frozen D-MTP source."""

    def __init__(self, native: dict):
        super().__init__()
        D, eps = native["hidden_size"], native["rms_norm_eps"]
        self.pre_fc_norm_embedding = ZeroCenteredRMSNorm(D, eps)
        self.pre_fc_norm_hidden = ZeroCenteredRMSNorm(D, eps)
        self.fc = Linear(2 * D, D)
        self.midlayer = MTPDecoderLayer(native)
        self.norm = ZeroCenteredRMSNorm(D, eps)

    def predict_embeddings(self, hidden, embeds, positions, intervals):
        """``hidden/embeds [T, D]`` packed rows; ``intervals [T, 4]`` causal same-document visibility."""
        x = self.fc(torch.cat((self.pre_fc_norm_embedding(embeds), self.pre_fc_norm_hidden(hidden)), -1))
        return self.norm(self.midlayer(x, positions, intervals))


def native_key(name: str) -> str:
    """Parameter name -> key inside the Target checkpoint."""
    return "mtp.layers.0." + name[len("midlayer."):] if name.startswith("midlayer.") else "mtp." + name


def causal_intervals(doc_start: torch.Tensor) -> torch.Tensor:
    t = torch.arange(doc_start.shape[0], device=doc_start.device)
    z = torch.zeros_like(t)
    return torch.stack([doc_start, t + 1, z, z], -1).to(torch.int32)


class NativeMTPDraftModel(MTPPredictor, Eagle3DraftModel):
    config_class = NativeMTPConfig

    def __init__(self, config):
        native = config.native_config
        Eagle3DraftModel.__init__(self)
        MTPPredictor.__init__(self, native)
        self.config = config
        self.native = native
        self.target_vocab_size = self.vocab_size = native["vocab_size"]
        self.embed_tokens = nn.Embedding(native["vocab_size"], native["hidden_size"])
        self.lm_head = Linear(native["hidden_size"], native["vocab_size"])
        self.norm_output = False
        self.draft_vocab_size = native["vocab_size"]
        self.embed_tokens.weight.requires_grad_(False)
        self.lm_head.weight.requires_grad_(False)

    native_key = staticmethod(native_key)

    @torch.no_grad()
    def initialize_native_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Copy only the native MTP tensors (``tensors`` maps Target checkpoint keys to tensors)."""
        for name, dest in self.state_dict().items():
            if name in ("embed_tokens.weight", "lm_head.weight"):
                continue
            src = tensors[native_key(name)]
            if src.shape != dest.shape:
                raise ValueError("Native MTP tensor shape mismatch: " + name)
            dest.copy_(src)

    @torch.no_grad()
    def validate_target_binding(self, embedding: torch.Tensor, lm_head: torch.Tensor) -> None:
        for name, expected in (("embed_tokens.weight", embedding), ("lm_head.weight", lm_head)):
            actual = self.state_dict()[name]
            if tuple(actual.shape) != tuple(expected.shape):
                raise ValueError("Native MTP shared Target tensor shape mismatch: " + name)
            for s in range(0, expected.shape[0], 1024):
                if not torch.equal(actual[s:s + 1024].cpu(), expected[s:s + 1024].to(actual.dtype).cpu()):
                    raise ValueError("Native MTP frozen tensor differs from its Target: " + name)

    def predict(self, hidden, input_ids, positions, intervals):
        return self.predict_embeddings(hidden, self.embed_tokens(input_ids).to(hidden.dtype), positions, intervals)

    def embed_input_ids(self, ids):
        return self.embed_tokens(ids)

    def project_hidden_states(self, hidden):
        return hidden

    def compute_logits(self, hidden):
        return self.lm_head(hidden)

    def backbone(self, *args, **kwargs):
        raise NotImplementedError("Native MTP uses predict(), not the EAGLE suffix recurrence")

    def get_lm_head_params(self):
        return None, self.lm_head.weight, self.native["rms_norm_eps"]

    def _serving_name(self, name: str) -> str:
        return ("model.embed_tokens.weight" if name == "embed_tokens.weight" else
                name if name == "lm_head.weight" else native_key(name))

    def state_dict_for_serving(self, state=None) -> dict:
        state = self.state_dict() if state is None else state
        return {self._serving_name(n): v for n, v in state.items()}

    def state_dict_from_serving(self, tensors: dict) -> dict:
        names = {self._serving_name(n): n for n in self.state_dict()}
        unknown = set(tensors) - set(names)
        if unknown:
            raise ValueError("Unknown native MTP serving tensors: " + str(sorted(unknown)))
        return {names[n]: v for n, v in tensors.items()}
