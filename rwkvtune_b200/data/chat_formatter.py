"""Jinja chat formatting and ShareGPT conversion (``rwkvtune/data/chat_formatter.py:9-153``)."""
from __future__ import annotations

import os
from typing import Dict, List, Optional

_DEFAULT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "chat_templates",
                        "rwkv_default.jinja")
_ROLE_MAP = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system"}


class ChatFormatter:
    def __init__(self, template_path: Optional[str] = None):
        from jinja2 import Template

        self.template_path = template_path or _DEFAULT
        with open(self.template_path, "r", encoding="utf-8") as fh:
            self.template_text = fh.read()
        self.template = Template(self.template_text)

    def format_messages(self, messages: List[Dict[str, str]], add_generation_prompt: bool = False, **kwargs) -> str:
        return self.template.render(messages=messages, add_generation_prompt=add_generation_prompt, **kwargs)

    @staticmethod
    def convert_sharegpt_to_messages(conversations: List[Dict[str, str]], system: Optional[str] = None) -> List[Dict[str, str]]:
        msgs = [{"role": "system", "content": system}] if system else []
        for turn in conversations:
            role = _ROLE_MAP.get(turn.get("from", turn.get("role", "")))
            if role is None:
                continue
            msgs.append({"role": role, "content": turn.get("value", turn.get("content", ""))})
        return msgs

    def format_sharegpt(self, conversations, system: Optional[str] = None, add_generation_prompt: bool = False) -> str:
        return self.format_messages(self.convert_sharegpt_to_messages(conversations, system), add_generation_prompt)

    def __repr__(self) -> str:
        return f"ChatFormatter(template={self.template_path})"


def get_default_formatter() -> ChatFormatter:
    return ChatFormatter()


def get_formatter(template_path: Optional[str] = None) -> ChatFormatter:
    return ChatFormatter(template_path)
