"""Model and generation configuration objects stored as JSON inside a hub directory.

Parity target: ``rwkvtune/models/configuration.py:12-268`` of the reference
(``RWKVConfig`` and ``GenerationConfig``).  The on-disk ``config.json`` keys are
identical so that hub directories written by either project load in the other.
Unknown keys survive a load/save round trip through ``_extra_config``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

CONFIG_NAME = "config.json"
GENERATION_CONFIG_NAME = "generation_config.json"


def _resolve_json(path: str, name: str) -> str:
    return os.path.join(path, name) if os.path.isdir(path) else path


@dataclass
class RWKVConfig:
    model_type: str = "rwkv7"
    architectures: List[str] = field(default_factory=lambda: ["RWKV7Model"])
    n_layer: int = 12
    n_embd: int = 768
    vocab_size: int = 65536
    head_size_a: int = 64
    ctx_len: int = 4096
    dim_att_lora: int = 64
    dim_gate_lora: int = 128
    dim_mv_lora: int = 32
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = 261
    pad_token_id: Optional[int] = 0
    dim_att: Optional[int] = None
    dim_ffn: Optional[int] = None
    head_size_divisor: int = 8
    my_testing: str = "x070"
    transformers_version: str = "rwkvtune-0.1.0"
    use_cache: bool = True
    tie_word_embeddings: bool = False
    _extra_config: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.dim_att is None:
            self.dim_att = self.n_embd
        if self.dim_ffn is None:
            # Kept for file compatibility only: the network itself uses 4 * n_embd.
            self.dim_ffn = int((self.n_embd * 3.5) // 32 * 32)

    # ------------------------------------------------------------------ derived
    @property
    def n_head(self) -> int:
        return self.dim_att // self.head_size_a

    @property
    def ffn_width(self) -> int:
        return 4 * self.n_embd

    # ------------------------------------------------------------------ (de)serialise
    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "RWKVConfig":
        data = config_dict
        known = {f.name for f in fields(cls)} - {"_extra_config"}
        kwargs = {k: v for k, v in data.items() if k in known}
        extra = {k: v for k, v in data.items() if k not in known}
        if extra:
            kwargs["_extra_config"] = extra
        return cls(**kwargs)

    @classmethod
    def from_json_file(cls, json_file: str) -> "RWKVConfig":
        with open(json_file, "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str) -> "RWKVConfig":
        path = pretrained_model_name_or_path
        cfg = _resolve_json(path, CONFIG_NAME)
        if not os.path.exists(cfg):
            raise FileNotFoundError(f"no {CONFIG_NAME} found at {path}")
        return cls.from_json_file(cfg)

    def to_dict(self) -> Dict[str, Any]:
        out = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "_extra_config"}
        out.update(self._extra_config)
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, ensure_ascii=False) + "\n"

    def to_json_file(self, json_file: str) -> None:
        with open(json_file, "w", encoding="utf-8") as fh:
            fh.write(self.to_json_string())

    def save_pretrained(self, save_directory: str) -> str:
        os.makedirs(save_directory, exist_ok=True)
        target = os.path.join(save_directory, CONFIG_NAME)
        with open(target, "w", encoding="utf-8") as fh:
            fh.write(self.to_json_string())
        return target

    def __getattr__(self, name: str) -> Any:
        # Attribute access falls through to the unknown keys captured at load time.
        extra = self.__dict__.get("_extra_config", {})
        if name in extra:
            return extra[name]
        raise AttributeError(name)

    def update(self, **kwargs: Any) -> "RWKVConfig":
        known = {f.name for f in fields(self)}
        for k, v in kwargs.items():
            if k in known:
                setattr(self, k, v)
            else:
                self._extra_config[k] = v
        return self


@dataclass
class GenerationConfig:
    """Sampling defaults saved as ``generation_config.json``
    (reference: ``rwkvtune/models/configuration.py:199-268``)."""

    eos_token_id: Optional[int] = 261
    pad_token_id: Optional[int] = 0
    bos_token_id: Optional[int] = None
    do_sample: bool = True
    temperature: float = 1.0
    top_p: float = 0.85
    top_k: int = 0
    repetition_penalty: float = 1.0
    max_length: int = 1024
    max_new_tokens: Optional[int] = None
    num_return_sequences: int = 1

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "GenerationConfig":
        data = config_dict
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in data.items() if k in known})

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str) -> "GenerationConfig":
        path = pretrained_model_name_or_path
        target = _resolve_json(path, GENERATION_CONFIG_NAME)
        if not os.path.exists(target):
            return cls()
        with open(target, "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    def to_dict(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_json_file(cls, json_file: str) -> "GenerationConfig":
        with open(json_file, "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    def to_json_file(self, json_file: str) -> None:
        with open(json_file, "w", encoding="utf-8") as fh:
            json.dump(self.to_dict(), fh, indent=2)
            fh.write("\n")

    def save_pretrained(self, save_directory: str) -> str:
        os.makedirs(save_directory, exist_ok=True)
        target = os.path.join(save_directory, GENERATION_CONFIG_NAME)
        with open(target, "w", encoding="utf-8") as fh:
            json.dump(self.to_dict(), fh, indent=2)
            fh.write("\n")
        return target
