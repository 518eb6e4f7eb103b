"""Create a hub directory (``config.json`` + weights + tokenizer files) from a bare weight file.

Layout and keys follow ``rwkvtune/utils/model_hub.py:15-541``: ``config.json``,
``generation_config.json``, ``tokenizer_config.json`` (with the chat template when given),
``vocab.txt``, ``model.pth`` or ``model.safetensors`` (copied, symlinked or converted) and a
``README.md``.  When no preset and no explicit sizes are given the architecture is inferred from
tensor shapes in the checkpoint.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Any, Dict, Optional

import torch

from ..configs import load_model_config
from ..data.tokenizers import TokenizerConfig, get_vocab_path
from ..models.configuration import GenerationConfig, RWKVConfig

_ARCH_KEYS = ("n_layer", "n_embd", "vocab_size", "head_size_a", "ctx_len", "dim_att_lora", "dim_gate_lora", "dim_mv_lora")


def _load_sd(path: str) -> Dict[str, torch.Tensor]:
    from ..models.auto_model import load_weight_file

    return load_weight_file(path)


def _extract_config_from_model(model_file: str) -> Optional[Dict[str, Any]]:
    """Infer the architecture from tensor shapes (``model_hub.py:276-327``)."""
    try:
        sd = _load_sd(model_file)
    except Exception:
        return None
    if "emb.weight" not in sd:
        return None
    vocab, C = sd["emb.weight"].shape
    layers = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("blocks."))
    out: Dict[str, Any] = {"n_layer": layers, "n_embd": int(C), "vocab_size": int(vocab)}
    rk = sd.get("blocks.0.att.r_k")
    if rk is not None and rk.ndim == 2:
        out["head_size_a"] = int(rk.shape[1])
    for key, name in (("dim_att_lora", "blocks.0.att.w1"), ("dim_gate_lora", "blocks.0.att.g1"),
                      ("dim_mv_lora", "blocks.1.att.v1")):
        if name in sd:
            out[key] = int(sd[name].shape[1])
    return out


def _convert_weight_format(source_file: str, target_file: str) -> None:
    sd = {k: v.contiguous() for k, v in _load_sd(source_file).items()}
    if target_file.endswith(".safetensors"):
        from safetensors.torch import save_file

        save_file(sd, target_file)
    else:
        torch.save(sd, target_file)


def create_model_hub(output_dir: str, model_file: Optional[str] = None, config_name: Optional[str] = None,
                     config_dict: Optional[Dict[str, Any]] = None, vocab_file: Optional[str] = None,
                     chat_template_file: Optional[str] = None, model_name: Optional[str] = None,
                     description: Optional[str] = None, n_layer: Optional[int] = None, n_embd: Optional[int] = None,
                     vocab_size: Optional[int] = None, head_size_a: Optional[int] = None, ctx_len: Optional[int] = None,
                     dim_att_lora: Optional[int] = None, dim_gate_lora: Optional[int] = None,
                     dim_mv_lora: Optional[int] = None, temperature: float = 1.0, top_p: float = 0.85, top_k: int = 0,
                     repetition_penalty: float = 1.0, max_length: int = 1024, eos_token: str = "\n\n",
                     model_max_length: int = 4096, copy_weights: bool = True, save_format: str = "pth",
                     overwrite: bool = False) -> str:
    if os.path.exists(output_dir) and os.listdir(output_dir) and not overwrite:
        raise FileExistsError(f"{output_dir} exists and is not empty (pass overwrite=True)")
    arch: Dict[str, Any] = {}
    if config_name:
        arch.update(load_model_config(config_name).to_train_config_dict())
    elif model_file and not config_dict:
        arch.update(_extract_config_from_model(model_file) or {})
    if config_dict:
        arch.update({k: v for k, v in config_dict.items() if v is not None})
    overrides = dict(n_layer=n_layer, n_embd=n_embd, vocab_size=vocab_size, head_size_a=head_size_a, ctx_len=ctx_len,
                     dim_att_lora=dim_att_lora, dim_gate_lora=dim_gate_lora, dim_mv_lora=dim_mv_lora)
    arch.update({k: v for k, v in overrides.items() if v is not None})
    if "n_layer" not in arch or "n_embd" not in arch:
        raise ValueError("architecture unknown: give config_name, config_dict, n_layer/n_embd or a readable model_file")
    cfg = RWKVConfig.from_dict(arch)
    os.makedirs(output_dir, exist_ok=True)      # only once the architecture is known: a failed call leaves nothing
    cfg.save_pretrained(output_dir)
    GenerationConfig(temperature=temperature, top_p=top_p, top_k=top_k, repetition_penalty=repetition_penalty,
                     max_length=max_length).save_pretrained(output_dir)
    template = None
    if chat_template_file:
        with open(chat_template_file, "r", encoding="utf-8") as fh:
            template = fh.read()
        shutil.copyfile(chat_template_file, os.path.join(output_dir, "chat_template.jinja"))
    TokenizerConfig(vocab_file="vocab.txt", eos_token=eos_token, model_max_length=model_max_length,
                    chat_template=template).save_pretrained(output_dir)
    shutil.copyfile(vocab_file or get_vocab_path(), os.path.join(output_dir, "vocab.txt"))
    if model_file:
        ext = "safetensors" if save_format == "safetensors" else "pth"
        target = os.path.join(output_dir, f"model.{ext}")
        if os.path.lexists(target):
            os.remove(target)
        same_format = model_file.endswith(".safetensors") == (ext == "safetensors")
        if not same_format:
            _convert_weight_format(model_file, target)
        elif copy_weights:
            shutil.copyfile(model_file, target)
        else:
            os.symlink(os.path.abspath(model_file), target)
    _create_readme(output_dir, model_name or os.path.basename(os.path.normpath(output_dir)), description, cfg)
    return output_dir


def _create_readme(output_dir: str, model_name: str, description: Optional[str], cfg: RWKVConfig) -> None:
    lines = [f"# {model_name}", "", description or "RWKV-7 model directory.", "", "## Architecture", ""]
    lines += [f"- {k}: {getattr(cfg, k)}" for k in _ARCH_KEYS]
    lines += ["", "## Usage", "", "```python", "from rwkvtune_b200 import AutoModel, AutoTokenizer",
              f'model = AutoModel.from_pretrained("{output_dir}")', f'tokenizer = AutoTokenizer.from_pretrained("{output_dir}")',
              "```", ""]
    with open(os.path.join(output_dir, "README.md"), "w", encoding="utf-8") as fh:
        fh.write("\n".join(lines))
