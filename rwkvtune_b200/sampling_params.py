"""vLLM-style sampling parameters (``rwkvtune/sampling_params.py:10-79``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Union


@dataclass
class SamplingParams:
    max_tokens: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    stop: Optional[Union[str, List[str]]] = None
    stop_token_ids: Optional[List[int]] = None
    skip_special_tokens: bool = True
    repetition_penalty: float = 1.0
    logit_bias: Optional[Dict[int, float]] = None

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, got {self.max_tokens}")
        if self.temperature < 0:
            raise ValueError(f"temperature must be non-negative, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be non-negative, got {self.top_k}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be positive, got {self.repetition_penalty}")
        if isinstance(self.stop, str):
            self.stop = [self.stop]

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-6

    @classmethod
    def from_dict(cls, d: dict) -> "SamplingParams":
        """Unknown keys are ignored."""
        data = d
        known = cls.__dataclass_fields__
        return cls(**{key: value for key, value in data.items() if key in known})

    def to_dict(self) -> dict:
        from dataclasses import asdict

        return asdict(self)
