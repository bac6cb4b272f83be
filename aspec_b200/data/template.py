"""Chat templates: the strings that delimit turns, used both to format conversations and to locate assistant spans
for the loss mask (reference: aspec/data/template.py:26-330)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional


@dataclass(frozen=True)
class ChatTemplate:
    assistant_header: Optional[str]
    user_header: Optional[str]
    system_prompt: Optional[str]
    end_of_turn_token: Optional[str]
    parser_type: str = "general"          # general | thinking | harmony | tool_xml | kimi-k25 | minimax-m2
    enable_thinking: bool = False
    system_header: Optional[str] = None
    bos: str = ""
    image_placeholder: str = "<image>"


class TemplateRegistry:
    def __init__(self):
        self.templates: Dict[str, ChatTemplate] = {}

    def register(self, name: str, template: ChatTemplate, override: bool = False) -> None:
        if not override and name in self.templates:
            raise ValueError(f"Chat template for the model type {name} has already been registered")
        self.templates[name] = template

    def get(self, name: str) -> ChatTemplate:
        if name not in self.templates:
            raise KeyError(f"unknown chat template {name!r}; known: {sorted(self.templates)}")
        return self.templates[name]

    def get_all_template_names(self) -> List[str]:
        return list(self.templates)


TEMPLATE_REGISTRY = TemplateRegistry()
_IM = dict(assistant_header="<|im_start|>assistant\n", user_header="<|im_start|>user\n",
           system_header="<|im_start|>system\n", end_of_turn_token="<|im_end|>\n")
for _name, _tpl in {
    "llama3": ChatTemplate("<|start_header_id|>assistant<|end_header_id|>\n\n", "<|start_header_id|>user<|end_header_id|>\n\n",
                           "You are a helpful assistant.", "<|eot_id|>", system_header="<|start_header_id|>system<|end_header_id|>\n\n",
                           bos="<|begin_of_text|>"),
    "llama4": ChatTemplate("<|header_start|>assistant<|header_end|>\n\n", "<|header_start|>user<|header_end|>\n\n",
                           "You are a helpful assistant.", "<|eot|>", system_header="<|header_start|>system<|header_end|>\n\n"),
    "qwen": ChatTemplate(system_prompt="You are a helpful assistant.", **_IM),
    "qwen2-vl": ChatTemplate(system_prompt="You are a helpful assistant.", **_IM),
    "qwen3-thinking": ChatTemplate(system_prompt=None, parser_type="thinking", enable_thinking=True, **_IM),
    "qwen3-instruct": ChatTemplate(system_prompt=None, **_IM),
    "qwen3.5": ChatTemplate(system_prompt=None, parser_type="thinking", enable_thinking=True, **_IM),
    "ling": ChatTemplate("<role>ASSISTANT</role>", "<role>HUMAN</role>", None, "<|role_end|>", system_header="<role>SYSTEM</role>"),
    "phi3": ChatTemplate("<|assistant|>\n", "<|user|>\n", "You are a helpful assistant.", "<|end|>\n", system_header="<|system|>\n"),
    "phi4": ChatTemplate("<|im_start|>assistant<|im_sep|>", "<|im_start|>user<|im_sep|>", "You are a helpful assistant.",
                         "<|im_end|>", system_header="<|im_start|>system<|im_sep|>"),
    "deepseek-v3": ChatTemplate("<｜Assistant｜>", "<｜User｜>", None, "<｜end▁of▁sentence｜>", bos="<｜begin▁of▁sentence｜>"),
    "gpt-oss": ChatTemplate("<|start|>assistant", "<|start|>user<|message|>", None, "<|end|>", parser_type="harmony",
                            system_header="<|start|>system<|message|>"),
    "kimi-k2": ChatTemplate("<|im_assistant|>assistant<|im_middle|>", "<|im_user|>user<|im_middle|>", None, "<|im_end|>",
                            parser_type="tool_xml", system_header="<|im_system|>system<|im_middle|>"),
    "kimi-k2-thinking": ChatTemplate("<|im_assistant|>assistant<|im_middle|>", "<|im_user|>user<|im_middle|>", None, "<|im_end|>",
                                     parser_type="thinking", enable_thinking=True, system_header="<|im_system|>system<|im_middle|>"),
    "kimi-k25-vlm": ChatTemplate("<|im_assistant|>assistant<|im_middle|>", "<|im_user|>user<|im_middle|>", None, "<|im_end|>",
                                 parser_type="kimi-k25", system_header="<|im_system|>system<|im_middle|>",
                                 image_placeholder="<|image|>"),
    "minimax-m2": ChatTemplate("]~b]ai\n", "]~b]user\n", "You are a helpful assistant. Your name is MiniMax-M2.5 and is built by MiniMax.",
                               "[e~[", parser_type="minimax-m2", system_header="]~!b[]~b]system\n"),
}.items():
    TEMPLATE_REGISTRY.register(_name, _tpl)
