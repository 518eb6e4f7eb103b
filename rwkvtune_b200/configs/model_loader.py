"""Model-size presets: ``load_model_config("1.5b" | "rwkv7-1.5b" | path)``
(reference: ``rwkvtune/configs/model_loader.py:15-253``)."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "models")


class ModelConfig:
    def __init__(self, config_dict: Dict[str, Any], config_source: str = ""):
        self.raw, self.config_source = config_dict, config_source
        self.model_name = config_dict.get("model_name", "")
        self.description = config_dict.get("description", "")
        self.model_file = config_dict.get("model_file")
        arch = config_dict.get("architecture", {})
        self.n_layer, self.n_embd = arch.get("n_layer"), arch.get("n_embd")
        self.vocab_size = arch.get("vocab_size", 65536)
        self.head_size_a = arch.get("head_size_a", 64)
        self.ctx_len = arch.get("ctx_len", 4096)
        lora = config_dict.get("lora_dims", {})
        self.dim_att_lora = lora.get("dim_att_lora", 0)
        self.dim_gate_lora = lora.get("dim_gate_lora", 0)
        self.dim_mv_lora = lora.get("dim_mv_lora", 0)
        tr = config_dict.get("training", {})
        self.recommended_ctx_len = tr.get("recommended_ctx_len")
        self.recommended_batch_size = tr.get("recommended_batch_size")
        self.recommended_lr = tr.get("recommended_lr")
        self.architecture_version = config_dict.get("architecture_version", "rwkv7")

    @property
    def model_path(self) -> Optional[str]:
        return self.model_file if self.model_file and os.path.exists(self.model_file) else None

    def to_train_config_dict(self) -> Dict[str, Any]:
        return {k: getattr(self, k) for k in ("n_layer", "n_embd", "vocab_size", "head_size_a", "ctx_len",
                                              "dim_att_lora", "dim_gate_lora", "dim_mv_lora")}

    def to_rwkv_config(self):
        from ..models.configuration import RWKVConfig

        return RWKVConfig(**self.to_train_config_dict())

    def __repr__(self) -> str:
        return f"ModelConfig({self.model_name}: L{self.n_layer} D{self.n_embd} V{self.vocab_size})"


def list_available_models(config_dir: Optional[str] = None) -> Dict[str, str]:
    d = config_dir or _DIR
    return {f[:-5]: os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith(".json")} if os.path.isdir(d) else {}


def load_model_config(config_identifier: str, config_dir: Optional[str] = None,
                      default_arch: str = "rwkv7") -> ModelConfig:
    if os.path.isfile(config_identifier):
        path = config_identifier
    else:
        models = list_available_models(config_dir)
        key = config_identifier.lower()
        key = key if key in models else f"{default_arch}-{key}"
        if key not in models:
            raise ValueError(f"unknown model config {config_identifier!r}; available: {sorted(models)}")
        path = models[key]
    with open(path, "r", encoding="utf-8") as fh:
        return ModelConfig(json.load(fh), path)


def print_model_info(config: ModelConfig) -> None:
    print(f"{config.model_name}: {config.description}")
    for k, v in config.to_train_config_dict().items():
        print(f"  {k}: {v}")
    print(f"  recommended: ctx {config.recommended_ctx_len}, batch {config.recommended_batch_size}, lr {config.recommended_lr}")
