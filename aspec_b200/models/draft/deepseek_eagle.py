"""EAGLE3 draft with DeepSeek multi-head latent attention (reference: aspec/models/draft/deepseek_eagle.py:89-575)."""
from __future__ import annotations

import torch.nn as nn

from aspec_b200.config.draft_config import DeepseekEagleConfig
from aspec_b200.models.draft.llama3_eagle import LlamaForCausalLMEagle3
from aspec_b200.models.draft.mla import MLAAttention


class _MLAProjector(nn.Module):
    """Adapts ``MLAAttention`` to the EAGLE layer's ``project(x, positions)`` protocol (input width ``2D``)."""

    def __init__(self, config):
        super().__init__()
        self.mla = MLAAttention(config, input_width=2 * config.hidden_size)
        self.o_proj = self.mla.o_proj
        self.scale = self.mla.scale

    def project(self, x, positions):
        q = self.mla.queries(x, positions)
        k, v = self.mla.keys_values(x, positions)
        return q, k.contiguous(), v.contiguous()


class Eagle3DeepseekV2ForCausalLM(LlamaForCausalLMEagle3):
    config_class = DeepseekEagleConfig

    def __init__(self, config):
        super().__init__(config)
        self.midlayer.self_attn = _MLAProjector(config)
