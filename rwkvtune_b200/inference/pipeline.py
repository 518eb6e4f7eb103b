"""Single-model inference pipeline: load a hub directory or a raw ``.pth`` (architecture inferred from
tensor shapes or taken from a preset), then ``generate`` / ``chat``
(``rwkvtune/inference/pipeline.py:14-290``)."""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch

from ..models import AutoModel, RWKVConfig, RWKV7Model
from ..models.auto_model import load_weight_file, resolve_dtype
from .batch_generator import BatchGenerator, GenerationConfig


class InferencePipeline:
    def __init__(self, model_path: Optional[str] = None, model_config: Optional[str] = None, device: str = "cuda",
                 precision: str = "bf16", vocab_path: Optional[str] = None, debug_output: bool = False,
                 model=None, tokenizer=None):
        self.device = torch.device(device)
        self.precision = precision
        self.debug_output = debug_output
        dtype = resolve_dtype(precision) if self.device.type != "cpu" else torch.float32
        if model is not None:
            self.model = model.to(self.device)
        elif model_path and os.path.isdir(model_path):
            self.model = AutoModel.from_pretrained(model_path, device=self.device, dtype=dtype)
        else:
            arch = {}
            if model_config:
                from ..configs import load_model_config

                cfg_obj = load_model_config(model_config)
                arch = cfg_obj.to_train_config_dict()
                model_path = model_path or cfg_obj.model_path
            if not model_path:
                raise ValueError("model_path is required (directly or through a preset that names a weight file)")
            sd = load_weight_file(model_path)
            if not arch:
                from ..utils.model_hub import _extract_config_from_model

                arch = _extract_config_from_model(model_path) or {}
            self.model = RWKV7Model(RWKVConfig.from_dict(arch))
            self.model.load_state_dict(sd)
            self.model = self.model.to(device=self.device, dtype=dtype)
        self.model.eval()
        if tokenizer is not None:
            self.tokenizer = tokenizer
        elif model_path and os.path.isdir(model_path) and os.path.exists(os.path.join(model_path, "vocab.txt")):
            from ..data.tokenizers import AutoTokenizer

            self.tokenizer = AutoTokenizer.from_pretrained(model_path)
        else:
            from ..data.tokenizers import RWKVTokenizer, get_vocab_path

            self.tokenizer = RWKVTokenizer(vocab_path or get_vocab_path())
        self._generator = BatchGenerator(self.model, self.tokenizer, max_batch_size=8)

    def encode(self, text: str) -> List[int]:
        return self.tokenizer.encode(text)

    def decode(self, tokens: List[int]) -> str:
        return self.tokenizer.decode(tokens)

    def generate(self, prompt: str, max_tokens: int = 100, temperature: float = 1.0, top_p: float = 0.9,
                 top_k: int = 0, num_generations: int = 1, **kwargs):
        if top_p <= 0:          # the "greedy" preset
            temperature, top_p = 0.0, 1.0
        gc = GenerationConfig(max_length=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                              num_generations=num_generations)
        out = self._generator.generate(prompts=[prompt], generation_config=gc)
        if self.debug_output:
            print(f"[pipeline] prompt tokens {len(self.encode(prompt))}, generated {out['masks'].sum(-1).tolist()}")
        return out["completions"][0] if num_generations == 1 else out["completions"]

    def chat(self, user_input: str, history: Optional[List[Tuple[str, str]]] = None, max_tokens: int = 256,
             temperature: float = 1.0, top_p: float = 0.9) -> str:
        parts = [f"User: {u}\n\nAssistant: {a}\n\n" for u, a in (history or [])]
        parts.append(f"User: {user_input}\n\nAssistant:")
        text = self.generate("".join(parts), max_tokens=max_tokens, temperature=temperature, top_p=top_p)
        return text.strip()
