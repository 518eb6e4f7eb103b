"""vLLM-style result containers (``rwkvtune/outputs.py:10-67``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: List[int]
    cumulative_logprob: Optional[float] = None
    finish_reason: Optional[str] = None   # "stop" | "length"

    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class RequestOutput:
    request_id: str
    prompt: Optional[str]
    prompt_token_ids: List[int]
    outputs: List[CompletionOutput] = field(default_factory=list)
    finished: bool = True

    def __repr__(self) -> str:
        return (f"RequestOutput(request_id={self.request_id!r}, prompt={self.prompt!r}, "
                f"outputs={len(self.outputs)}, finished={self.finished})")
