"""Renderer that trusts the tokenizer's own ``apply_chat_template`` for the token stream and finds assistant spans
on token ids (header ... end-of-turn) with the native scan, instead of re-deriving the format from strings
(reference: aspec/data/renderers/kimi_k3.py:24-303).

The assistant header is derived by rendering a probe conversation twice (with and without the generation prompt)
and taking the difference; the tokenizer contract is checked once: the header must occur in a rendered assistant
turn and the end-of-turn token must follow the reply.
"""
from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch

from aspec_b200.data.loss_mask import compute_assistant_loss_mask

_PROBE = [{"role": "user", "content": "ping"}]
_END_CANDIDATES = ("<|im_end|>", "<|eot_id|>", "<|end|>", "<|role_end|>", "[e~[")


class K3Renderer:
    cache_version = "1"

    def __init__(self, tokenizer: Any):
        self.tokenizer = tokenizer
        with_prompt = self._template(_PROBE, add_generation_prompt=True)
        without = self._template(_PROBE, add_generation_prompt=False)
        if with_prompt[: len(without)] != without or len(with_prompt) <= len(without):
            raise ValueError("tokenizer chat template does not append an assistant header as generation prompt")
        self.header_ids = with_prompt[len(without):]
        self.end_ids = self._end_of_turn()
        probe = self._template(_PROBE + [{"role": "assistant", "content": "pong"}], add_generation_prompt=False)
        mask, _ = compute_assistant_loss_mask(torch.tensor(probe), self.header_ids, self.end_ids)
        if int(mask.sum()) == 0:
            raise ValueError("tokenizer contract violated: no assistant span found in a rendered assistant turn")

    def _template(self, messages, tools=None, add_generation_prompt=False, **kw) -> List[int]:
        ids = self.tokenizer.apply_chat_template(messages, tools=tools, tokenize=True,
                                                 add_generation_prompt=add_generation_prompt, **kw)
        if isinstance(ids, dict):
            ids = ids["input_ids"]
        if hasattr(ids, "tolist"):
            ids = ids.tolist()
        if ids and isinstance(ids[0], list):
            ids = ids[0]
        return [int(i) for i in ids]

    def _end_of_turn(self) -> List[int]:
        vocab = getattr(self.tokenizer, "get_vocab", lambda: {})()
        for tok in _END_CANDIDATES:
            if tok in vocab:
                return [int(vocab[tok])]
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is None:
            raise ValueError("cannot determine the end-of-turn token of this tokenizer")
        return [int(eos)]

    def get_assistant_token_ids(self) -> Tuple[List[int], List[int], int]:
        return list(self.header_ids), list(self.end_ids), 0

    def render(self, messages: List[dict], tools: Optional[List[dict]] = None, max_seq_length: Optional[int] = None,
               last_turn_only: bool = False, generation_config: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        from aspec_b200.data.parse import normalize_conversation
        kwargs = dict(generation_config or {})
        messages = [{k: v for k, v in m.items() if not k.startswith("_")} for m in normalize_conversation(messages)]
        ids = self._template(messages, tools=tools, add_generation_prompt=False, **kwargs)
        if max_seq_length:
            ids = ids[:max_seq_length]
        t = torch.tensor(ids, dtype=torch.long)
        mask, _ = compute_assistant_loss_mask(t, self.header_ids, self.end_ids, last_turn_only=last_turn_only)
        # the end-of-turn token belongs to the reply: supervise it too
        ends = (mask[:-1] == 1) & (mask[1:] == 0)
        mask[1:][ends] = 1
        return t, mask.long()
