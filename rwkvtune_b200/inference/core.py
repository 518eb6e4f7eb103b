"""Token sampling.

One rule set for every caller (the reference's single-row ``sample`` and batched ``sample_batch``
disagree on the top-p boundary; ``rwkvtune/inference/core.py:120-123`` vs ``:219-224``): ids above
the tokenizer's largest id are banned; ``temperature < 1e-6`` is greedy; then temperature,
``logit_bias`` (clamped to +-100), an optional ``logits_processor``, top-k, and top-p keeping the
sorted prefix with ``cumsum <= top_p`` plus always the most likely token.  Returns the sampled ids
and their log-probabilities under the filtered distribution.

On CUDA the whole rule - repetition penalty from a seen-token bitmap, ban, temperature or greedy, bias, top-k,
top-p, draw, log-probability - runs in one launch of the ``rwkv_sample_tokens`` kernel (threshold searches over the
row instead of a full 65536-way sort) unless a ``logits_processor`` is given; everything stays on the device.  A
``torch.Generator`` or an explicit ``seed`` makes draws reproducible.
"""
from __future__ import annotations

import warnings
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.nn.functional as F


def apply_repetition_penalty(logits: torch.Tensor, seen_mask: torch.Tensor, penalty: float) -> torch.Tensor:
    """``seen_mask`` is a ``[B, V]`` bool bitmap of tokens already present in each row's history."""
    if penalty is None or penalty == 1.0 or penalty <= 0:
        return logits
    scaled = torch.where(logits > 0, logits / penalty, logits * penalty)
    return torch.where(seen_mask, scaled, logits)


class TokenSampler:
    _max_valid_token_id: Optional[int] = None
    use_native_kernel: bool = True

    @classmethod
    def set_max_valid_token_id(cls, max_id: Optional[int]) -> None:
        cls._max_valid_token_id = max_id

    @staticmethod
    def filter_logits(logits: torch.Tensor, temperature: float, top_p: float, top_k: int,
                      logit_bias: Optional[Dict] = None, logits_processor: Optional[Callable] = None,
                      max_valid_token_id: Optional[int] = None) -> torch.Tensor:
        """Banned ids, temperature, bias, processor, top-k and top-p applied; masked entries are ``-inf``."""
        logits = logits.float().clone()
        V = logits.shape[-1]
        mv = max_valid_token_id if max_valid_token_id is not None else TokenSampler._max_valid_token_id
        if mv is not None:
            if mv + 1 < V:
                logits[..., mv + 1:] = float("-inf")
            elif mv >= V:
                warnings.warn(f"max_valid_token_id ({mv}) >= logits width ({V}): tokenizer/model vocabulary mismatch")
        if temperature >= 1e-6 and temperature != 1.0:
            logits = logits / temperature
        if logit_bias:
            for tid, bias in logit_bias.items():
                tid = int(tid)
                if 0 <= tid < V:
                    logits[..., tid] += min(100.0, max(-100.0, float(bias)))
        if logits_processor is not None:
            logits = logits_processor(logits)
        if temperature < 1e-6:
            return logits
        if top_k and top_k > 0:
            kth = torch.topk(logits, min(top_k, V), dim=-1).values[..., -1:]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        if top_p < 1.0:
            sl, si = torch.sort(logits, descending=True, dim=-1)
            cum = torch.cumsum(F.softmax(sl, dim=-1), dim=-1)
            keep = cum <= top_p
            keep[..., 0] = True
            sl = sl.masked_fill(~keep, float("-inf"))
            logits = torch.full_like(logits, float("-inf")).scatter(-1, si, sl)
        return logits

    @staticmethod
    def sample_batch(logits_batch: torch.Tensor, temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0,
                     logit_bias: Optional[Dict] = None, logits_processor: Optional[Callable] = None,
                     generator: Optional[torch.Generator] = None, seed: Optional[int] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
        if logits_batch.dim() != 2:
            raise ValueError(f"batch sampling needs 2-D logits, got shape {tuple(logits_batch.shape)}")
        if logits_batch.is_cuda and TokenSampler.use_native_kernel and logits_processor is None:
            from . import sampling_native

            if sampling_native.full_available() and logits_batch.shape[1] <= 65536:
                return sampling_native.sample_tokens(logits_batch, temperature, top_p, top_k, logit_bias,
                                                     TokenSampler._max_valid_token_id, seed=seed, generator=generator)
        filtered = TokenSampler.filter_logits(logits_batch, temperature, top_p, top_k, logit_bias, logits_processor)
        logp = F.log_softmax(filtered, dim=-1)
        if temperature < 1e-6:
            tokens = filtered.argmax(dim=-1)
        else:
            probs = logp.exp()
            bad = ~torch.isfinite(probs).all(dim=-1) | (probs.sum(-1) <= 0)
            if bool(bad.any()):   # NaN/Inf rows fall back to a uniform draw over valid ids
                probs = torch.where(bad[:, None], torch.ones_like(probs), torch.nan_to_num(probs, nan=0.0, posinf=0.0))
            if seed is not None and generator is None:
                generator = torch.Generator(device=probs.device).manual_seed(int(seed))
            tokens = torch.multinomial(probs, 1, generator=generator).squeeze(-1)
        return tokens, logp.gather(1, tokens[:, None]).squeeze(1)

    @staticmethod
    def sample(logits: torch.Tensor, temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0,
               logit_bias: Optional[Dict] = None, logits_processor: Optional[Callable] = None,
               generator: Optional[torch.Generator] = None) -> Tuple[int, float]:
        tok, lp = TokenSampler.sample_batch(logits.reshape(1, -1), temperature, top_p, top_k, logit_bias,
                                            logits_processor, generator)
        return int(tok[0]), float(lp[0])
