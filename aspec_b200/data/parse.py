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


def _flatten_content(content: Any, image_text: str) -> str:
    """Message content as text: a string, or a list of ``{"type": "text" | "image" | "image_url", ...}`` parts where
    every image part becomes ``image_text``."""
    if isinstance(content, str):
        return content
    if isinstance(content, (list, tuple)):
        return "".join(part.get("text", "") if part.get("type") == "text" else
                       image_text if part.get("type") in ("image", "image_url") else "" for part in content)
    return "" if content is None else str(content)


def _split_reasoning(text: str) -> Tuple[str, str]:
    """``(reasoning, answer)`` of a reply that may hold one ``<think>`` block (whose opener may be missing)."""
    if "</think>" not in text:
        return "", text
    head, tail = text.split("</think>", 1)
    return head.split("<think>")[-1].strip("\n"), tail.strip("\n")


class _DialectParser(Parser):
    """Parsers whose turn syntax is fixed by the model family rather than by a template's header strings.

    A subclass states the wire format as data (``ROLE_OPEN``, ``TURN_CLOSE``, ``IMAGE``) and writes one assistant turn in
    ``_assistant_turn``; walking the conversation, image expansion, history trimming and the loss-mask pattern are shared.
    ``expand_media_tokens=False`` keeps the dataset's image placeholder in the text (for a later multimodal processor).
    """

    ROLE_OPEN: Dict[str, str] = {}
    TURN_CLOSE = ""
    IMAGE = ""
    PROMPT_OPEN = ""           # what follows the assistant header when a generation prompt is requested

    def __init__(self, tokenizer, chat_template):
        super().__init__(tokenizer, chat_template)
        self.placeholder = chat_template.image_placeholder or "<image>"
        self.assistant_pattern = re.escape(self.ROLE_OPEN["assistant"]) + r"(.*?" + re.escape(self.TURN_CLOSE) + r"|.*\Z)"

    def _text_of(self, msg: Dict[str, Any], expand: bool) -> str:
        image = (self.IMAGE + "\n") if expand else self.placeholder
        text = _flatten_content(msg.get("content"), image)
        if expand and isinstance(msg.get("content"), str) and msg["role"] == "user":
            text = text.replace(self.placeholder, self.IMAGE + "\n")
        return text

    def _raw_messages(self, conversation) -> Conversation:
        out = []
        for msg in conversation:
            role = msg.get("role", msg.get("from"))
            if role not in _ROLES:
                raise ValueError(f"unknown message role {role!r}")
            out.append({**msg, "role": _ROLES[role], "content": msg.get("content", msg.get("value"))})
        return out

    def format(self, conversation, last_turn_only: bool = False, add_generation_prompt: bool = False,
               expand_media_tokens: bool = True) -> str:
        msgs = self._raw_messages(conversation)
        pieces = self._walk(msgs, expand_media_tokens)
        if add_generation_prompt:
            pieces.append(self.ROLE_OPEN["assistant"] + self.PROMPT_OPEN)
        return "".join(pieces)


class KimiK25Parser(_DialectParser):
    """Kimi-K2.5 (reference behaviour: aspec/data/parse.py:380-536).  No default system prompt; every assistant turn
    opens with a ``<think>`` block (empty when there is no reasoning); only the last assistant turn keeps its reasoning;
    tool calls use the family's inline section tokens; a tool result is a system-side ``tool`` turn."""

    ROLE_OPEN = {"system": "<|im_system|>system<|im_middle|>", "user": "<|im_user|>user<|im_middle|>",
                 "assistant": "<|im_assistant|>assistant<|im_middle|>", "tool": "<|im_system|>tool<|im_middle|>"}
    TURN_CLOSE = "<|im_end|>"
    IMAGE = "<|media_begin|>image<|media_content|><|media_pad|><|media_end|>"
    PROMPT_OPEN = "<think>"

    @staticmethod
    def _calls(calls) -> str:
        body = "".join(f"<|tool_call_begin|>{c.get('id', '')}<|tool_call_argument_begin|>"
                       f"{c.get('function', {}).get('arguments', '')}<|tool_call_end|>" for c in calls)
        return "<|tool_calls_section_begin|>" + body + "<|tool_calls_section_end|>"

    def _walk(self, msgs, expand):
        final = max((i for i, m in enumerate(msgs) if m["role"] == "assistant"), default=-1)
        out = []
        for i, m in enumerate(msgs):
            text = self._text_of(m, expand)
            if m["role"] == "assistant":
                if "</think>" in text and "<think>" not in text:          # opener eaten by a generation prompt
                    text = "<think>" + text
                if i != final:
                    text = _THINK.sub("", text)
                elif m.get("reasoning_content") and "<think>" not in text:
                    text = f"<think>{str(m['reasoning_content']).strip()}</think>{text}"
                if m.get("tool_calls"):
                    text += self._calls(m["tool_calls"])
                if not text.startswith("<think>"):
                    text = "<think></think>" + text
            elif m["role"] == "tool" and m.get("tool_call_id"):
                text = f"## Return of {m['tool_call_id']}\n{text}"
            out.append(self.ROLE_OPEN[m["role"]] + text + self.TURN_CLOSE)
        return out


class MiniMaxParser(_DialectParser):
    """MiniMax-M2 (reference behaviour: aspec/data/parse.py:539-700).  A system turn always opens the text; reasoning is
    kept only in assistant turns after the last user message (interleaved thinking); tool calls are
    ``<minimax:tool_call>`` XML; consecutive tool results share one ``tool`` turn."""

    ROLE_OPEN = {"system": "]~!b[]~b]system\n", "user": "]~b]user\n", "assistant": "]~b]ai\n", "tool": "]~b]tool"}
    TURN_CLOSE = "[e~["
    IMAGE = "]<]start of image[>[]<]vision pad[>[]<]end of image[>["
    PROMPT_OPEN = "<think>\n"
    DEFAULT_SYSTEM = "You are a helpful assistant."

    @staticmethod
    def _calls(calls) -> str:
        blocks = []
        for call in calls:
            fn = call.get("function", call)
            args = fn.get("arguments", {})
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except ValueError:
                    args = {"raw": args}
            lines = [f'<invoke name="{fn.get("name", "")}">']
            for key, value in (args.items() if isinstance(args, dict) else ()):
                shown = value if isinstance(value, str) else json.dumps(value, ensure_ascii=False)
                lines.append(f'<parameter name="{key}">{shown}</parameter>')
            blocks.append("\n".join(lines + ["</invoke>"]))
        return "\n<minimax:tool_call>\n" + "\n".join(blocks) + "\n</minimax:tool_call>"

    def _walk(self, msgs, expand):
        if msgs and msgs[0]["role"] == "system":
            system, msgs = self._text_of(msgs[0], expand), msgs[1:]
        else:
            system = self.template.system_prompt or self.DEFAULT_SYSTEM
        out = [self.ROLE_OPEN["system"] + system + self.TURN_CLOSE + "\n"]
        last_user = max((i for i, m in enumerate(msgs) if m["role"] == "user"), default=-1)
        for i, m in enumerate(msgs):
            text = self._text_of(m, expand)
            if m["role"] == "assistant":
                reasoning = m.get("reasoning_content") or ""
                if not reasoning:
                    reasoning, text = _split_reasoning(text)
                turn = (f"<think>\n{reasoning}\n</think>\n\n" if reasoning and i > last_user else "") + text
                if m.get("tool_calls"):
                    turn += self._calls(m["tool_calls"])
                out.append(self.ROLE_OPEN["assistant"] + turn + self.TURN_CLOSE + "\n")
            elif m["role"] == "tool":
                opens = i == 0 or msgs[i - 1]["role"] != "tool"
                closes = i == len(msgs) - 1 or msgs[i + 1]["role"] != "tool"
                out.append((self.ROLE_OPEN["tool"] if opens else "") + f"\n<response>{text}</response>"
                           + (self.TURN_CLOSE + "\n" if closes else ""))
            else:
                out.append(self.ROLE_OPEN[m["role"]] + text + self.TURN_CLOSE + "\n")
        return out


_PARSERS = {"general": GeneralParser, "thinking": ThinkingParser, "harmony": HarmonyParser, "tool_xml": ToolXMLParser,
            "kimi-k25": KimiK25Parser, "minimax-m2": MiniMaxParser}


def create_parser(tokenizer, chat_template: ChatTemplate) -> Parser:
    if chat_template.parser_type not in _PARSERS:
        raise ValueError(f"unknown parser type {chat_template.parser_type!r}")
    return _PARSERS[chat_template.parser_type](tokenizer, chat_template)
