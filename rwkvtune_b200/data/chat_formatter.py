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
    def convert_sharegpt_to_messages(conversations: List[Dict[str, str]], include_gpt_ignore: bool = True,
                                     system: Optional[str] = None) -> List[Dict[str, str]]:
        """``gpt_ignore`` turns (assistant text that takes no loss) are kept as assistant messages flagged
        ``_ignore`` when ``include_gpt_ignore``, dropped otherwise (``rwkvtune/data/chat_formatter.py:73-112``)."""
        msgs = [{"role": "system", "content": system}] if system else []
        for turn in conversations:
            src = turn.get("from", turn.get("role", ""))
            content = turn.get("value", turn.get("content", ""))
            if src == "gpt_ignore":
                if include_gpt_ignore:
                    msgs.append({"role": "assistant", "content": content, "_ignore": True})
                continue
            role = _ROLE_MAP.get(src)
            if role is None:
                continue
            msgs.append({"role": role, "content": content})
        return msgs

    def format_sharegpt(self, conversations, add_generation_prompt: bool = False, include_gpt_ignore: bool = True,
                        system: Optional[str] = None) -> str:
        return self.format_messages(self.convert_sharegpt_to_messages(conversations, include_gpt_ignore, system),
                                    add_generation_prompt)

    def __repr__(self) -> str:
        return f"ChatFormatter(template={self.template_path})"


def get_default_formatter() -> ChatFormatter:
    return ChatFormatter()


def get_formatter(template_path: Optional[str] = None) -> ChatFormatter:
    return ChatFormatter(template_path)
