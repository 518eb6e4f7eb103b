"""Offline batch generation on the continuous-batching scheduler
(``rwkvtune/inference/batch_generator.py:28-244``): ``generate(prompts | input_ids, GenerationConfig)``
returns completions with a trailing EOS stripped, 0-padded ids and float masks."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from .scheduler_core import SchedulerCore, SequenceState


@dataclass
class GenerationConfig:
    max_length: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    num_generations: int = 1
    max_batch_tokens: int = 8192
    chunk_size: int = 512


class BatchGenerator:
    def __init__(self, model, tokenizer, config=None, use_state_cache: bool = False, max_batch_size: int = 64,
                 verbose: bool = False, **kwargs):
        self.model, self.tokenizer = model, tokenizer
        self.device = next(model.parameters()).device
        self.default_config = config or GenerationConfig()
        self.eos_id = getattr(tokenizer, "eos_token_id", None)
        self.verbose = verbose
        cache = None
        if use_state_cache:
            from .state_cache import create_state_cache

            cache = create_state_cache(model, kwargs.get("max_cache_memory_gb", 4.0))
        self.state_cache = cache
        self.scheduler = SchedulerCore(model, tokenizer, max_batch_size, self.default_config.max_batch_tokens,
                                       self.default_config.chunk_size, cache)

    @torch.no_grad()
    def generate(self, prompts: Optional[List[str]] = None, generation_config: Optional[GenerationConfig] = None,
                 input_ids: Optional[List[List[int]]] = None) -> Dict[str, Any]:
        gc = generation_config or self.default_config
        if input_ids is None:
            if prompts is None:
                raise ValueError("provide prompts or input_ids")
            input_ids = [self.tokenizer.encode(p) for p in prompts]
        was_training = self.model.training
        self.model.eval()
        G = gc.num_generations
        total = len(input_ids) * G
        sched = self.scheduler
        sched.max_batch_tokens, sched.prefill_chunk_size = gc.max_batch_tokens, gc.chunk_size
        sched.reset()
        seqs = [SequenceState(seq_id=i * G + g, prompt_tokens=list(ids), max_new_tokens=gc.max_length,
                              temperature=gc.temperature, top_p=gc.top_p, top_k=gc.top_k, eos_token_id=self.eos_id)
                for i, ids in enumerate(input_ids) for g in range(G)]
        sched.add_sequences(seqs)
        for _ in sched.run_to_completion_sync():
            pass
        if was_training:
            self.model.train()
        return self._postprocess([list(s.generated_tokens) for s in seqs], total, gc)

    def _postprocess(self, all_tokens: List[List[int]], total: int, gc: GenerationConfig) -> Dict[str, Any]:
        completions, eos_stops, len_stops = [], 0, 0
        for i, toks in enumerate(all_tokens):
            if len(toks) >= gc.max_length:
                len_stops += 1
            if self.eos_id is not None and toks and toks[-1] == self.eos_id:
                toks = all_tokens[i] = toks[:-1]
                eos_stops += 1
            completions.append(self.tokenizer.decode(toks) if self.tokenizer is not None else "")
        if self.verbose and all_tokens:
            lens = [len(t) for t in all_tokens]
            print(f"[BatchGenerator] {len(lens)} sequences, length mean {sum(lens) / len(lens):.1f} "
                  f"min {min(lens)} max {max(lens)}, eos {eos_stops}, max_length {len_stops}")
        max_len = max((len(t) for t in all_tokens), default=0)
        ids = torch.zeros(total, max_len, dtype=torch.long, device=self.device)
        masks = torch.zeros(total, max_len, dtype=torch.float32, device=self.device)
        for i, t in enumerate(all_tokens):
            if t:
                ids[i, :len(t)] = torch.tensor(t, dtype=torch.long, device=self.device)
                masks[i, :len(t)] = 1.0
        return {"completions": completions, "completion_ids": ids,
                "completion_logps": torch.tensor([], device=self.device), "masks": masks}
