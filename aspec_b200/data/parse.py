"""Conversation -> (token ids, loss mask).  A parser formats the messages with a chat template and marks the
assistant replies (header excluded, end-of-turn token included) as supervised
(reference: aspec/data/parse.py:82-720).

The mask is computed on characters and mapped to tokens by encoding prefixes, which is exact for any tokenizer whose
encoding of a prefix ending at a template boundary is a prefix of the full encoding (all special-token delimited
templates).  ``thinking`` templates keep ``<think>`` blocks of the supervised turns and drop them from earlier turns;
``harmony`` templates supervise every assistant channel message; ``tool_xml`` templates serialise tool calls inside
the assistant turn.
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Sequence, Tuple

import torch

from aspec_b200.data.template import ChatTemplate

Conversation = List[Dict[str, Any]]
_THINK = re.compile(r"<think>.*?</think>\s*", re.S)
_ROLES = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system",
          "tool": "tool", "function": "tool", "observation": "tool"}


def normalize_conversation(conversation: Sequence[Dict[str, Any]]) -> Conversation:
    """Accepts ``role/content`` and ShareGPT ``from/value`` messages."""
    out = []
    for msg in conversation:
        role = msg.get("role", msg.get("from"))
        if role not in _ROLES:
            raise ValueError(f"unknown message role {role!r}")
        item = {"role": _ROLES[role], "content": msg.get("content", msg.get("value")) or ""}
        for key in ("tool_calls", "reasoning_content", "name", "_done"):
            if msg.get(key):
                item[key] = msg[key]
        out.append(item)
    return out


def has_thinking_content(conversation: Sequence[Dict[str, Any]]) -> bool:
    return any(m.get("role") == "assistant" and ("<think>" in (m.get("content") or "") or m.get("reasoning_content"))
               for m in conversation)


def has_unbalanced_thinking_tags(text: str) -> bool:
    return text.count("<think>") != text.count("</think>")


class Parser:
    def __init__(self, tokenizer, chat_template: ChatTemplate):
        self.tokenizer = tokenizer
        self.template = chat_template
        end = re.escape(chat_template.end_of_turn_token or "")
        self.assistant_pattern = re.escape(chat_template.assistant_header or "") + r"(.*?" + (end if end else r"\Z") + r"|.*\Z)"

    # -- formatting -------------------------------------------------------------------------------------------
    def _assistant_text(self, msg: Dict[str, Any], supervised: bool) -> str:
        return msg["content"]

    def format(self, conversation: Conversation, last_turn_only: bool = False) -> str:
        t = self.template
        msgs = normalize_conversation(conversation)
        parts = [t.bos]
        if msgs and msgs[0]["role"] == "system":
            system, msgs = msgs[0]["content"], msgs[1:]
        else:
            system = t.system_prompt
        if system and t.system_header is not None:
            parts.append(t.system_header + system + (t.end_of_turn_token or ""))
        elif system and t.user_header is not None and t.system_header is None:
            msgs = [{**msgs[0], "content": system + "\n\n" + msgs[0]["content"]}] + msgs[1:] if msgs else msgs
        last_assistant = max((i for i, m in enumerate(msgs) if m["role"] == "assistant"), default=-1)
        for i, m in enumerate(msgs):
            if m["role"] == "assistant":
                supervised = (not last_turn_only) or i == last_assistant
                parts.append((t.assistant_header or "") + self._assistant_text(m, supervised) + (t.end_of_turn_token or ""))
            else:
                body = m["content"] if m["role"] == "user" else self._tool_text(m)
                parts.append((t.user_header or "") + body + (t.end_of_turn_token or ""))
        return "".join(parts)

    def _tool_text(self, msg: Dict[str, Any]) -> str:
        return "<tool_response>\n" + str(msg["content"]) + "\n</tool_response>"

    # -- tokenisation -------------------------------------------------------------------------------------------
    def _encode(self, text: str) -> List[int]:
        return list(self.tokenizer.encode(text, add_special_tokens=False))

    def tokenize_with_loss_mask(self, text: str, max_length: int, last_turn_only: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        ids = self._encode(text)[:max_length]
        mask = torch.zeros(len(ids), dtype=torch.long)
        matches = list(re.finditer(self.assistant_pattern, text, re.S))
        if last_turn_only and matches:
            matches = matches[-1:]
        for m in matches:
            start = min(len(self._encode(text[: m.start(1)])), len(ids))
            end = min(len(self._encode(text[: m.end(1)])), len(ids))
            if start < end:
                mask[start:end] = 1
        return torch.tensor(ids, dtype=torch.long), mask

    def parse(self, conversation: Conversation, max_length: int, preformatted: bool = False, last_turn_only: bool = False):
        text = conversation if preformatted else self.format(conversation, last_turn_only=last_turn_only)
        return self.tokenize_with_loss_mask(text, max_length, last_turn_only)


class GeneralParser(Parser):
    pass


class ThinkingParser(Parser):
    """Reasoning stays in supervised turns and is dropped from history turns (what serving engines replay)."""

    def _assistant_text(self, msg, supervised):
        content = msg["content"]
        if msg.get("_done"):
            return content
        reasoning = msg.get("reasoning_content")
        if reasoning and "<think>" not in content:
            content = f"<think>\n{reasoning.strip()}\n</think>\n\n{content}"
        if "</think>" in content and "<think>" not in content:      # opener consumed by a generation prompt
            content = "<think>" + content
        if not supervised:
            return _THINK.sub("", content)
        if self.template.enable_thinking and "<think>" not in content:
            content = "<think>\n\n</think>\n\n" + content
        return content

    def format(self, conversation, last_turn_only: bool = False):
        # only the turns after the last user message keep their reasoning, whatever the loss covers
        msgs = normalize_conversation(conversation)
        last_user = max((i for i, m in enumerate(msgs) if m["role"] == "user"), default=-1)
        msgs = [({**m, "content": self._assistant_text(m, i > last_user), "reasoning_content": None, "_done": True}
                 if m["role"] == "assistant" else m) for i, m in enumerate(msgs)]
        return Parser.format(self, msgs, last_turn_only=last_turn_only)


class HarmonyParser(Parser):
    """``<|start|>assistant<|channel|>NAME<|message|>...<|end|>``; analysis (reasoning) and final channels."""

    def __init__(self, tokenizer, chat_template):
        super().__init__(tokenizer, chat_template)
        self.assistant_pattern = (re.escape("<|start|>assistant<|channel|>") + r"\w+" + re.escape("<|message|>")
                                  + r"(.*?(?:" + re.escape("<|end|>") + "|" + re.escape("<|return|>") + r")|.*\Z)")

    def _assistant_text(self, msg, supervised):
        out = ""
        reasoning = msg.get("reasoning_content")
        if reasoning and supervised:
            out += f"<|channel|>analysis<|message|>{reasoning}<|end|><|start|>assistant"
        return out + f"<|channel|>final<|message|>{msg['content']}"


class ToolXMLParser(ThinkingParser):
    """Assistant tool calls are serialised as ``<tool_call>{json}</tool_call>`` lines inside the turn."""

    def _assistant_text(self, msg, supervised):
        text = super()._assistant_text(msg, supervised)
        for call in msg.get("tool_calls") or []:
            fn = call.get("function", call)
            args = fn.get("arguments")
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except json.JSONDecodeError:
                    pass
            text += "\n<tool_call>\n" + json.dumps({"name": fn.get("name"), "arguments": args}, ensure_ascii=False) + "\n</tool_call>"
        return text


_PARSERS = {"general": GeneralParser, "thinking": ThinkingParser, "harmony": HarmonyParser, "tool_xml": ToolXMLParser}


def create_parser(tokenizer, chat_template: ChatTemplate) -> Parser:
    if chat_template.parser_type not in _PARSERS:
        raise ValueError(f"unknown parser type {chat_template.parser_type!r}")
    return _PARSERS[chat_template.parser_type](tokenizer, chat_template)
