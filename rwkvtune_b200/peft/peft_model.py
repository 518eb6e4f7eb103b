"""Apply, save, load and merge LoRA adapters (``rwkvtune/peft/peft_model.py:16-352``).

``get_peft_model`` replaces every ``nn.Linear`` whose qualified name contains one of
``config.target_modules`` (for RWKV-7: ``att.receptance/key/value/output`` and ``ffn.key/value``;
``head`` is not matched), freezes everything, then unfreezes the adapters and every parameter whose
name contains a ``modules_to_save`` entry (``["ln", "time"]`` -> all LayerNorm / GroupNorm weights).
The helper methods the reference monkey-patches onto the model are attached here as well.
"""
from __future__ import annotations

import json
import os
import types
from pathlib import Path
from typing import Dict, Optional, Union

import torch
import torch.nn as nn

from .config import LoraConfig
from .lora.layer import LoraLinear

ADAPTER_CONFIG = "adapter_config.json"
LEGACY_CONFIG = "lora_config.json"
ADAPTER_WEIGHTS = ("adapter_model.bin", "adapter_model.safetensors", "lora_weights.pth")


def is_peft_model(model: nn.Module) -> bool:
    return bool(getattr(model, "_is_peft_model", False)) or any(isinstance(m, LoraLinear) for m in model.modules())


def _lora_layers(model: nn.Module):
    return [(n, m) for n, m in model.named_modules() if isinstance(m, LoraLinear)]


def get_peft_model(model: nn.Module, peft_config: LoraConfig) -> nn.Module:
    config = peft_config
    targets = list(config.target_modules)
    replaced = 0
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if isinstance(child, nn.Linear) and not isinstance(child, LoraLinear) and any(t in full for t in targets):
                setattr(module, child_name, LoraLinear(child, config.r, config.lora_alpha, config.lora_dropout,
                                                       config.use_rslora, config.init_lora_weights))
                replaced += 1
    if replaced == 0:
        raise ValueError(f"no nn.Linear matched target_modules={targets}")
    for name, p in model.named_parameters():
        p.requires_grad = ("lora_A" in name or "lora_B" in name
                           or any(key in name for key in (config.modules_to_save or [])))
    model._is_peft_model = True
    model.peft_config = config
    _attach_methods(model)
    return model


# ----------------------------------------------------------------------------------- attached methods
def _disable_adapter(self):
    for _, m in _lora_layers(self):
        m.disable_adapter()


def _enable_adapter(self):
    for _, m in _lora_layers(self):
        m.enable_adapter()


def _merge_adapter(self):
    for _, m in _lora_layers(self):
        m.merge()


def _unmerge_adapter(self):
    for _, m in _lora_layers(self):
        m.unmerge()


def _get_lora_state_dict(self) -> Dict[str, torch.Tensor]:
    return {k: v.detach().cpu() for k, v in self.state_dict().items() if "lora_" in k}


def _get_trainable_extra_state_dict(self) -> Dict[str, torch.Tensor]:
    """Trained non-adapter parameters (the ``modules_to_save`` ones), by their own names."""
    out = {}
    for name, p in self.named_parameters():
        if p.requires_grad and "lora_" not in name:
            out[name.replace(".base_layer.", ".")] = p.detach().cpu()
    return out


def _get_merged_state_dict(self) -> Dict[str, torch.Tensor]:
    """Plain state_dict with adapters folded in: ``.base_layer.`` stripped, ``lora_*`` dropped.

    Nothing in the model is modified: each merged matrix ``W + s B A`` is formed on the side.  Base weights that are
    sharded across ranks (ZeRO-3 keeps only a column panel of each frozen matrix per rank and leaves an empty tensor
    in the module) are first reassembled from the panels."""
    sd = {k: v for k, v in self.state_dict().items() if "lora_A" not in k and "lora_B" not in k}
    for name, m in _lora_layers(self):
        key = f"{name}.base_layer.weight"
        sw = getattr(m, "_sharded", None)
        base = sw.full_weight() if sw is not None else m.base_layer.weight
        if m.merged:
            sd[key] = base.detach()
            continue
        delta = (m.lora_B.detach().float() @ m.lora_A.detach().float()) * m.scaling
        sd[key] = (base.detach().float() + delta.to(base.device)).to(base.dtype)
    for name, m in self.named_modules():   # sharded matrices that carry no adapter
        sw = getattr(m, "_sharded", None)
        if sw is not None and not isinstance(m, LoraLinear):
            sd[f"{name}.weight"] = sw.full_weight().detach()
    return {k.replace(".base_layer.", "."): v.detach().cpu().clone() for k, v in sd.items()}


def _save_lora_weights(self, path: str) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    sd = _get_lora_state_dict(self)
    sd.update(_get_trainable_extra_state_dict(self))
    torch.save(sd, path)


def _load_lora_weights(self, path: str, strict: bool = False):
    if str(path).endswith(".safetensors"):
        from safetensors.torch import load_file

        sd = load_file(str(path))
    else:
        sd = torch.load(str(path), map_location="cpu", weights_only=False)
    if isinstance(sd, dict) and "lora_state_dict" in sd:
        sd = sd["lora_state_dict"]
    own = self.state_dict()
    alias = {k.replace(".base_layer.", "."): k for k in own}
    loaded, skipped = 0, []
    with torch.no_grad():
        for k, v in sd.items():
            k2 = k[6:] if k.startswith("model.") else k
            target = k2 if k2 in own else alias.get(k2)
            if target is None or own[target].shape != v.shape:
                skipped.append(k)
                continue
            own[target].copy_(v.to(device=own[target].device, dtype=own[target].dtype))
            loaded += 1
    if strict and skipped:
        raise KeyError(f"adapter keys without a destination: {skipped[:5]}")
    return loaded, skipped


def _attach_methods(model: nn.Module) -> None:
    for name, fn in (("disable_adapter", _disable_adapter), ("enable_adapter", _enable_adapter),
                     ("merge_adapter", _merge_adapter), ("unmerge_adapter", _unmerge_adapter),
                     ("get_lora_state_dict", _get_lora_state_dict), ("get_merged_state_dict", _get_merged_state_dict),
                     ("get_trainable_extra_state_dict", _get_trainable_extra_state_dict),
                     ("save_lora_weights", _save_lora_weights), ("load_lora_weights", _load_lora_weights)):
        setattr(model, name, types.MethodType(fn, model))


def load_peft_model(model: nn.Module, peft_model_path: Union[str, Path], adapter_name: str = "default") -> nn.Module:
    d = Path(peft_model_path)
    if not d.exists():
        raise ValueError(f"LoRA directory does not exist: {d}")
    cfg_file = next((d / n for n in (ADAPTER_CONFIG, LEGACY_CONFIG) if (d / n).exists()), None)
    if cfg_file is None:
        raise ValueError(f"no {ADAPTER_CONFIG} or {LEGACY_CONFIG} in {d}")
    with open(cfg_file, "r", encoding="utf-8") as fh:
        c = json.load(fh)
    cfg = LoraConfig(r=c.get("r", 64), lora_alpha=c.get("lora_alpha", 128), lora_dropout=c.get("lora_dropout", 0.0),
                     target_modules=c.get("target_modules"), modules_to_save=c.get("modules_to_save"),
                     use_rslora=c.get("use_rslora", False))
    model = get_peft_model(model, cfg)
    weights = next((d / n for n in ADAPTER_WEIGHTS if (d / n).exists()), None)
    if weights is None:
        raise ValueError(f"no adapter weights ({', '.join(ADAPTER_WEIGHTS)}) in {d}")
    model.load_lora_weights(str(weights))
    return model
