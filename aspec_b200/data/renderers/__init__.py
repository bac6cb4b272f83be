"""Conversation renderers: chat messages -> (token ids, loss mask) through the tokenizer's own chat template
(text processing on the CPU).  Selected with ``dataset.renderer`` (reference: aspec/data/renderers/)."""
from aspec_b200.data.renderers.base import ConversationRenderer
from aspec_b200.data.renderers.registry import RENDERER_REGISTRY, RendererRegistry

__all__ = ["ConversationRenderer", "RENDERER_REGISTRY", "RendererRegistry"]
