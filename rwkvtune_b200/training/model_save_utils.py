"""Saving models and adapters in the hub-directory format
(``rwkvtune/training/model_save_utils.py:26-311``).

Differences from the reference, both deliberate: a ``lora_only`` save also stores the trained
non-adapter parameters (the LayerNorm / GroupNorm weights unfrozen by ``modules_to_save``) under
their own keys, which the reference drops; a ``full`` save of a LoRA model writes clean merged keys
instead of ``...base_layer.weight`` plus ``lora_*``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch

from ..peft import is_peft_model

WEIGHTS_NAME = "model.pth"
ADAPTER_WEIGHTS_NAME = "adapter_model.bin"


def _cpu_state_dict(model) -> Dict[str, torch.Tensor]:
    return {k: v.detach().cpu().contiguous() for k, v in model.state_dict().items()}


def save_tokenizer(tokenizer, output_dir: str) -> None:
    if tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
        tokenizer.save_pretrained(output_dir)


def save_model_with_config(model, output_dir: str, tokenizer=None, save_format: str = "pth",
                           state_dict: Optional[Dict[str, torch.Tensor]] = None, dtype: Optional[torch.dtype] = None) -> str:
    os.makedirs(output_dir, exist_ok=True)
    if hasattr(model, "config") and hasattr(model.config, "save_pretrained"):
        model.config.save_pretrained(output_dir)
    sd = state_dict if state_dict is not None else _cpu_state_dict(model)
    if dtype is not None:
        sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    if save_format == "safetensors":
        from safetensors.torch import save_file

        path = os.path.join(output_dir, "model.safetensors")
        save_file({k: v.contiguous() for k, v in sd.items()}, path)
    else:
        path = os.path.join(output_dir, WEIGHTS_NAME)
        torch.save(sd, path)
    save_tokenizer(tokenizer, output_dir)
    return path


def save_model_checkpoint(module, save_directory: str, checkpoint_name: str, tokenizer=None,
                          model_path: Optional[str] = None) -> str:
    """Weights + config (+ tokenizer) under ``save_directory/checkpoint_name``
    (``rwkvtune/training/model_save_utils.py:116-140``).  ``module`` is a model or anything holding one as
    ``.model`` (a trainer, an engine); ``model_path`` is accepted for signature parity and not needed."""
    model = getattr(module, "model", module)
    return save_model_with_config(model, os.path.join(save_directory, checkpoint_name), tokenizer=tokenizer,
                                  save_format="pth")


def get_lora_state_dict(model_or_sd) -> Dict[str, torch.Tensor]:
    sd = model_or_sd if isinstance(model_or_sd, dict) else model_or_sd.state_dict()
    out = {}
    for k, v in sd.items():
        if "lora_" in k:
            out[k[6:] if k.startswith("model.") else k] = v.detach().cpu()
    return out


def save_lora_checkpoint(model, output_dir: str, tokenizer=None, base_model_name_or_path: str = "") -> str:
    os.makedirs(output_dir, exist_ok=True)
    sd = get_lora_state_dict(model)
    if hasattr(model, "get_trainable_extra_state_dict"):
        sd.update(model.get_trainable_extra_state_dict())
    path = os.path.join(output_dir, ADAPTER_WEIGHTS_NAME)
    torch.save(sd, path)
    cfg = getattr(model, "peft_config", None)
    body: Dict[str, Any] = {"peft_type": "LORA", "base_model_name_or_path": base_model_name_or_path,
                            "task_type": "CAUSAL_LM", "inference_mode": True}
    if cfg is not None:
        body.update(cfg.to_dict())
    for name in ("adapter_config.json", "lora_config.json"):
        with open(os.path.join(output_dir, name), "w", encoding="utf-8") as fh:
            json.dump(body, fh, indent=2)
    if hasattr(model, "config") and hasattr(model.config, "save_pretrained"):
        model.config.save_pretrained(output_dir)
    save_tokenizer(tokenizer, output_dir)
    return path


def save_checkpoint_with_lora_support(model, output_dir: str, tokenizer=None, lora_save_mode: str = "lora_only",
                                      base_model_name_or_path: str = "", dtype: Optional[torch.dtype] = None) -> None:
    """Plain models: full save.  LoRA models: ``lora_only`` -> adapter files, ``full`` -> merged weights,
    ``both`` -> adapter files plus merged weights in ``<dir>/merged``."""
    if not is_peft_model(model):
        save_model_with_config(model, output_dir, tokenizer, dtype=dtype)
        return
    if lora_save_mode in ("lora_only", "both"):
        save_lora_checkpoint(model, output_dir, tokenizer, base_model_name_or_path)
    if lora_save_mode in ("full", "both"):
        target = output_dir if lora_save_mode == "full" else os.path.join(output_dir, "merged")
        save_model_with_config(model, target, tokenizer, state_dict=model.get_merged_state_dict(), dtype=dtype)
