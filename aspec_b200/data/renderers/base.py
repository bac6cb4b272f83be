"""Renderer protocol (reference: aspec/data/renderers/base.py:27-70)."""
from __future__ import annotations

from typing import List, Optional, Protocol, Tuple, runtime_checkable

import torch


@runtime_checkable
class ConversationRenderer(Protocol):
    cache_version: str

    def get_assistant_token_ids(self) -> Tuple[List[int], List[int], int]:
        """``(assistant header ids, end-of-turn ids, tokens to skip after the header)``."""

    def render(self, messages: List[dict], tools: Optional[List[dict]] = None, max_seq_length: Optional[int] = None,
               last_turn_only: bool = False, generation_config: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Token ids and a 0/1 loss mask of equal length."""
