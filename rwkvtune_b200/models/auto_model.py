"""``AutoModel``: build a model from a hub directory or a bare weight file.

Behavioural parity with ``rwkvtune/models/auto_model.py:58-223``: a directory is
searched for ``model.pth`` / ``pytorch_model.pth`` / ``model.safetensors``; a file
takes ``config.json`` from its own directory; ``{"model": state_dict}`` wrappers
are unwrapped; loading is non-strict by default.  Two deliberate differences:
weights are loaded *before* the dtype cast (so an fp32 checkpoint is rounded once,
not twice) and parameter initialisation is vectorised.
"""
from __future__ import annotations

import os
from typing import Optional, Union

import torch

from .configuration import RWKVConfig

MODEL_MAPPING = {"rwkv7": "RWKV7Model"}
WEIGHT_FILE_CANDIDATES = ("model.pth", "pytorch_model.pth", "model.safetensors")
_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32,
    "float16": torch.float16, "fp16": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
}


def resolve_dtype(dtype: Optional[Union[str, torch.dtype]]) -> Optional[torch.dtype]:
    if dtype is None or isinstance(dtype, torch.dtype):
        return dtype
    return _DTYPES.get(str(dtype).lower(), torch.float32)


def load_weight_file(path: str):
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file

        return load_file(path)
    sd = torch.load(path, map_location="cpu", weights_only=False)
    if isinstance(sd, dict) and "model" in sd and isinstance(sd["model"], dict):
        sd = sd["model"]
    return sd


class AutoModel:
    @staticmethod
    def _get_model_class(model_type: str):
        if model_type not in MODEL_MAPPING:
            raise ValueError(f"unsupported model_type {model_type!r}; supported: {sorted(MODEL_MAPPING)}")
        from .rwkv7 import RWKV7Model

        return RWKV7Model

    @classmethod
    def from_config(cls, config: RWKVConfig, **kwargs):
        return cls._get_model_class(config.model_type)(config, **kwargs)

    @classmethod
    def from_pretrained(cls, model_path: str, device: Optional[Union[str, torch.device]] = "cpu",
                        dtype: Optional[Union[str, torch.dtype]] = None, **kwargs):
        if os.path.isdir(model_path):
            config_dir, weight_file = model_path, None
            for name in WEIGHT_FILE_CANDIDATES:
                cand = os.path.join(model_path, name)
                if os.path.exists(cand):
                    weight_file = cand
                    break
        elif os.path.isfile(model_path):
            weight_file = model_path
            config_dir = os.path.dirname(model_path) or "."
        else:
            raise ValueError(f"path does not exist: {model_path} (expected a model directory or a .pth file)")
        config = RWKVConfig.from_pretrained(config_dir)
        model = cls.from_config(config)
        if kwargs.pop("load_weights", True):
            if weight_file is None:
                raise FileNotFoundError(
                    f"no weight file in {config_dir}; looked for {', '.join(WEIGHT_FILE_CANDIDATES)}")
            kwargs.pop("strict", False)
            model.load_state_dict(load_weight_file(weight_file), strict=False)
        dt = resolve_dtype(dtype)
        if dt is not None:
            model = model.to(dtype=dt)
        if device is not None:
            model = model.to(device)
        return model

    @classmethod
    def save_pretrained(cls, model, save_directory: str, save_format: str = "pth", **kwargs) -> str:
        os.makedirs(save_directory, exist_ok=True)
        if hasattr(model, "config"):
            model.config.save_pretrained(save_directory)
        sd = {k: v.detach().cpu().contiguous() for k, v in model.state_dict().items()}
        if save_format == "safetensors":
            from safetensors.torch import save_file

            target = os.path.join(save_directory, "model.safetensors")
            save_file(sd, target)
        else:
            target = os.path.join(save_directory, "model.pth")
            torch.save(sd, target)
        return target
