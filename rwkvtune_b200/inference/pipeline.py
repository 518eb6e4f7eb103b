"""Single-model inference pipeline: load a hub directory or a raw ``.pth`` (architecture inferred from
tensor shapes or taken from a preset), then ``generate`` / ``chat``
(``rwkvtune/inference/pipeline.py:14-290``)."""
from __future__ import annotations

import os
from typing import List, Optional, Tuple, Union

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

    def generate(self, prompt: Union[str, List[str]], max_tokens: int = 100, temperature: float = 1.0,
                 top_p: float = 0.9, top_k: int = 0, num_generations: int = 1, stream: bool = False, **kwargs):
        """One prompt or a list of prompts (``rwkvtune/inference/pipeline.py:198-255``).  A single prompt with
        ``num_generations=1`` returns a string; every other case returns a list, prompt-major
        (``len(prompt) * num_generations`` entries).  ``stream`` only prints each finished completion."""
        single = isinstance(prompt, str)
        prompts = [prompt] if single else list(prompt)
        if top_p <= 0:          # the "greedy" preset
            temperature, top_p = 0.0, 1.0
        gc = GenerationConfig(max_length=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                              num_generations=num_generations)
        out = self._generator.generate(prompts=prompts, generation_config=gc)
        if self.debug_output:
            print(f"[pipeline] prompt tokens {[len(self.encode(p)) for p in prompts]}, "
                  f"generated {out['masks'].sum(-1).tolist()}")
        completions = out["completions"]
        if stream:
            for text in completions:
                print(text, flush=True)
        return completions[0] if single and num_generations == 1 else completions

    def chat(self, user_input: str, system_prompt: Optional[str] = None,
             history: Optional[List[Tuple[str, str]]] = None, **kwargs) -> str:
        """``history`` is a list of ``(user, assistant)`` turns; keyword arguments go to :meth:`generate`
        (defaults: 256 new tokens)."""
        parts = [f"System: {system_prompt}\n\n"] if system_prompt else []
        parts += [f"User: {u}\n\nAssistant: {a}\n\n" for u, a in (history or [])]
        parts.append(f"User: {user_input}\n\nAssistant:")
        kwargs.setdefault("max_tokens", 256)
        return self.generate("".join(parts), **kwargs).strip()
