"""LoRA configuration (``rwkvtune/peft/config.py:56-128``)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Union

RWKV7_DEFAULT_TARGET_MODULES = ["receptance", "key", "value", "output", "key_ffn", "value_ffn"]


@dataclass
class LoraConfig:
    r: int = 64
    lora_alpha: int = 128
    lora_dropout: float = 0.0
    target_modules: Optional[Union[List[str], str]] = None
    modules_to_save: Optional[List[str]] = None
    use_rslora: bool = False
    init_lora_weights: Union[bool, str] = True

    def __post_init__(self) -> None:
        if self.r <= 0:
            raise ValueError(f"`r` must be a positive integer, got {self.r}")
        if self.target_modules is None:
            self.target_modules = list(RWKV7_DEFAULT_TARGET_MODULES)
        elif isinstance(self.target_modules, str):
            self.target_modules = {"att": ["receptance", "key", "value", "output"],
                                   "ffn": ["key_ffn", "value_ffn"]}.get(self.target_modules, [self.target_modules])
        if self.modules_to_save is None:
            self.modules_to_save = ["ln", "time"]

    @property
    def scaling(self) -> float:
        return self.lora_alpha / math.sqrt(self.r) if self.use_rslora else self.lora_alpha / self.r

    def to_dict(self) -> dict:
        return {"r": self.r, "lora_alpha": self.lora_alpha, "lora_dropout": self.lora_dropout,
                "target_modules": list(self.target_modules), "modules_to_save": list(self.modules_to_save),
                "use_rslora": self.use_rslora}
