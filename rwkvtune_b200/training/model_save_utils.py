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
    """``model.state_dict()`` on the CPU.  Matrices that ZeRO-3 holds as one column panel per rank are reassembled
    (the reference consolidates a stage-3 run into one ``model.pth`` the same way,
    ``rwkvtune/training/callbacks.py:385-426``)."""
    sd = {k: v.detach().cpu().contiguous() for k, v in model.state_dict().items()}
    for name, m in model.named_modules():
        sw = getattr(m, "_sharded", None)
        if sw is not None:
            key = f"{name}.base_layer.weight" if hasattr(m, "base_layer") else f"{name}.weight"
            sd[key] = sw.full_weight().detach().cpu().contiguous()
    return sd


def save_tokenizer(tokenizer, output_dir: str) -> None:
    if tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
        tokenizer.save_pretrained(output_dir)


def save_model_with_config(model, save_directory: str, model_name: str = "model", tokenizer=None, model_config_obj=None,
                           save_format: str = "pth", is_main_process: bool = True,
                           state_dict: Optional[Dict[str, torch.Tensor]] = None,
                           dtype: Optional[torch.dtype] = None) -> Optional[str]:
    """``config.json`` + ``<model_name>.pth`` / ``.safetensors`` (+ tokenizer files) in ``save_directory``
    (``rwkvtune/training/model_save_utils.py:26-113``).  ``model`` is a module or a state dict; the config comes from
    ``model_config_obj`` or ``model.config``; ranks other than the main one do nothing."""
    if not is_main_process:
        return None
    output_dir = save_directory
    os.makedirs(output_dir, exist_ok=True)
    cfg = model_config_obj if model_config_obj is not None else getattr(model, "config", None)
    if cfg is not None and hasattr(cfg, "save_pretrained"):
        cfg.save_pretrained(output_dir)
    if state_dict is not None:
        sd = state_dict
    elif isinstance(model, dict):
        sd = {k: v.detach().cpu() for k, v in model.items()}
    else:
        sd = _cpu_state_dict(model)
    if dtype is not None:
        sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    if save_format == "safetensors":
        from safetensors.torch import save_file

        path = os.path.join(output_dir, f"{model_name}.safetensors")
        save_file({k: v.contiguous() for k, v in sd.items()}, path)
    else:
        path = os.path.join(output_dir, WEIGHTS_NAME if model_name == "model" else f"{model_name}.pth")
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


def get_lora_state_dict(model) -> Dict[str, torch.Tensor]:
    """The ``lora_`` entries of a module's (or a state dict's) parameters, on the CPU."""
    sd = model if isinstance(model, dict) else model.state_dict()
    out = {}
    for k, v in sd.items():
        if "lora_" in k:
            out[k[6:] if k.startswith("model.") else k] = v.detach().cpu()
    return out


def save_lora_checkpoint(model, save_directory: str, lora_config: Optional[Dict[str, Any]] = None,
                         base_model_path: Optional[str] = None, tokenizer=None, safe_serialization: bool = False,
                         is_main_process: bool = True) -> Optional[str]:
    """Adapter weights + ``adapter_config.json`` (``rwkvtune/training/model_save_utils.py:154-237``).  The adapter
    settings come from ``model.peft_config``; entries of ``lora_config`` (a dict) override them.  With
    ``safe_serialization`` the weights go to ``adapter_model.safetensors``."""
    if not is_main_process:
        return None
    output_dir, base_model_name_or_path = save_directory, base_model_path or ""
    os.makedirs(output_dir, exist_ok=True)
    sd = get_lora_state_dict(model)
    if hasattr(model, "get_trainable_extra_state_dict"):
        sd.update(model.get_trainable_extra_state_dict())
    if safe_serialization:
        from safetensors.torch import save_file

        path = os.path.join(output_dir, "adapter_model.safetensors")
        save_file({k: v.contiguous() for k, v in sd.items()}, path)
    else:
        path = os.path.join(output_dir, ADAPTER_WEIGHTS_NAME)
        torch.save(sd, path)
    cfg = getattr(model, "peft_config", None)
    body: Dict[str, Any] = {"peft_type": "LORA", "base_model_name_or_path": base_model_name_or_path,
                            "task_type": "CAUSAL_LM", "inference_mode": True}
    if cfg is not None:
        body.update(cfg.to_dict())
    if lora_config:
        body.update(lora_config)
    for name in ("adapter_config.json", "lora_config.json"):
        with open(os.path.join(output_dir, name), "w", encoding="utf-8") as fh:
            json.dump(body, fh, indent=2)
    if hasattr(model, "config") and hasattr(model.config, "save_pretrained"):
        model.config.save_pretrained(output_dir)
    save_tokenizer(tokenizer, output_dir)
    return path


def save_model_or_adapter(model, output_dir: str, tokenizer=None, lora_save_mode: str = "lora_only",
                          base_model_name_or_path: str = "", dtype: Optional[torch.dtype] = None) -> None:
    """What the trainers call.  Plain models: full save.  LoRA models: ``lora_only`` -> adapter files, ``full`` ->
    merged weights, ``both`` -> adapter files plus merged weights in ``<dir>/merged``."""
    if not is_peft_model(model):
        save_model_with_config(model, output_dir, tokenizer=tokenizer, dtype=dtype)
        return
    if lora_save_mode in ("lora_only", "both"):
        save_lora_checkpoint(model, output_dir, base_model_path=base_model_name_or_path, tokenizer=tokenizer)
    if lora_save_mode in ("full", "both"):
        target = output_dir if lora_save_mode == "full" else os.path.join(output_dir, "merged")
        save_model_with_config(model, target, tokenizer=tokenizer, state_dict=model.get_merged_state_dict(), dtype=dtype)


def save_checkpoint_with_lora_support(lightning_module, save_directory: str, checkpoint_name: str, tokenizer=None,
                                      model_path: Optional[str] = None, use_lora: bool = False,
                                      lora_save_mode: str = "lora_only", lora_config: Optional[Dict[str, Any]] = None,
                                      is_main_process: bool = True) -> Optional[str]:
    """The reference's entry point (``rwkvtune/training/model_save_utils.py:240-330``): saves under
    ``save_directory/checkpoint_name``; ``lightning_module`` is a model or an object holding one as ``.model``.
    ``use_lora`` is implied by the model itself; ``lora_config`` entries override the stored adapter settings."""
    if not is_main_process:
        return None
    model = getattr(lightning_module, "model", lightning_module)
    target = os.path.join(save_directory, checkpoint_name)
    save_model_or_adapter(model, target, tokenizer, lora_save_mode, model_path or "")
    if lora_config and is_peft_model(model) and lora_save_mode in ("lora_only", "both"):
        save_lora_checkpoint(model, target, lora_config=lora_config, base_model_path=model_path, tokenizer=None)
    return target
