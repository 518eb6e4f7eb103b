"""Preset-driven text generation and a small REPL (``rwkvtune/inference/generator.py:9-145``)."""
from __future__ import annotations

from typing import List, Optional, Tuple

from .pipeline import InferencePipeline


class TextGenerator:
    PRESETS = {
        "greedy": {"temperature": 1.0, "top_p": 0.0, "top_k": 0},
        "creative": {"temperature": 0.8, "top_p": 0.9, "top_k": 0},
        "precise": {"temperature": 0.3, "top_p": 0.5, "top_k": 0},
        "balanced": {"temperature": 0.6, "top_p": 0.8, "top_k": 0},
    }

    def __init__(self, pipeline: InferencePipeline):
        self.pipeline = pipeline

    def generate(self, prompt: str, preset: str = "balanced", max_tokens: int = 100, **kwargs) -> str:
        if preset not in self.PRESETS:
            raise ValueError(f"unknown preset {preset!r}; available: {list(self.PRESETS)}")
        return self.pipeline.generate(prompt, max_tokens=max_tokens, **{**self.PRESETS[preset], **kwargs})

    def complete(self, prompt: str, max_tokens: int = 50, n: int = 1, **kwargs) -> List[str]:
        """``n`` independent completions of ``prompt`` (``rwkvtune/inference/generator.py:69-95``)."""
        result = self.pipeline.generate(prompt, max_tokens=max_tokens, num_generations=n, **kwargs)
        return result if isinstance(result, list) else [result]

    def interactive_chat(self, system_prompt: Optional[str] = None, input_fn=input, max_turns: Optional[int] = None) -> None:
        history: List[Tuple[str, str]] = []
        if system_prompt:
            print(f"System: {system_prompt}")
        turns = 0
        while max_turns is None or turns < max_turns:
            try:
                user = input_fn("User: ").strip()
            except (EOFError, KeyboardInterrupt):
                break
            if user.lower() in ("quit", "exit"):
                break
            if user.lower() == "clear":
                history.clear()
                continue
            if not user:
                continue
            reply = self.pipeline.chat(user, system_prompt=system_prompt, history=history)
            print(f"Assistant: {reply}")
            history.append((user, reply))
            turns += 1
