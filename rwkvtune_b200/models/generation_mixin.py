"""``generate()`` for any model exposing ``forward_with_state``.

Same keyword surface and stopping rules as ``rwkvtune/models/generation_mixin.py:31-225``
(one prefill, then single-token steps; stop once every row has produced an EOS id;
rows that finished early keep receiving sampled tokens until then).  Unlike the
reference there is no per-token host loop: repetition penalty uses a ``[B, V]``
seen-token mask kept on the device and the only host synchronisation per step is
the "all rows finished" check.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

import torch


def apply_repetition_penalty_(logits: torch.Tensor, seen: torch.Tensor, penalty: float) -> None:
    """Divide positive / multiply negative logits of already-seen tokens by ``penalty``, in place."""
    if penalty is None or penalty == 1.0 or penalty <= 0:
        return
    scaled = torch.where(logits > 0, logits / penalty, logits * penalty)
    logits.copy_(torch.where(seen, scaled, logits))


def sample_from_logits(logits: torch.Tensor, do_sample: bool, temperature: float, top_k: int, top_p: float,
                       generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Greedy / temperature / top-k / top-p draw from ``[B, V]`` fp32 logits.

    Top-p keeps the smallest prefix of the sorted distribution whose mass reaches
    ``top_p`` (the token that crosses the threshold is kept), as the reference's
    ``generate`` does (``generation_mixin.py:185-194``).
    """
    if not do_sample or temperature == 0:
        return torch.argmax(logits, dim=-1)
    if temperature > 0 and temperature != 1.0:
        logits = logits / temperature
    probs = torch.softmax(logits, dim=-1)
    if top_k and top_k > 0:
        kth = torch.topk(probs, min(top_k, probs.shape[-1]), dim=-1).values[..., -1:]
        probs = torch.where(probs < kth, torch.zeros_like(probs), probs)
        probs = probs / probs.sum(-1, keepdim=True)
    if 0 < top_p < 1.0:
        sp, si = torch.sort(probs, descending=True, dim=-1)
        cum = torch.cumsum(sp, dim=-1)
        remove = cum > top_p
        remove[..., 1:] = remove[..., :-1].clone()
        remove[..., 0] = False
        sp = sp.masked_fill(remove, 0.0)
        probs = torch.zeros_like(probs).scatter_(-1, si, sp)
        probs = probs / probs.sum(-1, keepdim=True)
    return torch.multinomial(probs, 1, generator=generator).squeeze(1)


class GenerationMixin:
    @torch.no_grad()
    def generate(
        self,
        input_ids: Optional[torch.Tensor] = None,
        inputs: Optional[torch.Tensor] = None,
        max_new_tokens: Optional[int] = None,
        max_length: Optional[int] = None,
        min_length: Optional[int] = None,
        do_sample: bool = True,
        temperature: float = 1.0,
        top_k: int = 0,
        top_p: float = 1.0,
        repetition_penalty: float = 1.0,
        num_return_sequences: int = 1,
        eos_token_id: Optional[Union[int, List[int]]] = None,
        pad_token_id: Optional[int] = None,
        token_ban: Optional[List[int]] = None,
        return_dict_in_generate: bool = False,
        output_scores: bool = False,
        initial_states: Optional[List[Dict[str, Any]]] = None,
        generator: Optional[torch.Generator] = None,
        **kwargs: Any,
    ):
        if input_ids is None:
            input_ids = inputs
        if input_ids is None:
            raise ValueError("generate() needs input_ids (or inputs)")
        if input_ids.dim() == 1:
            input_ids = input_ids.unsqueeze(0)
        B, T0 = input_ids.shape
        if max_new_tokens is not None:
            budget = int(max_new_tokens)
        elif max_length is not None:
            budget = int(max_length) - T0
        else:
            budget = 512
        if eos_token_id is None:
            eos_token_id = getattr(getattr(self, "config", None), "eos_token_id", None)
        eos_ids = [] if eos_token_id is None else ([eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id))
        if num_return_sequences > 1:
            input_ids = input_ids.repeat_interleave(num_return_sequences, dim=0)
            if initial_states is not None:
                initial_states = [{k: v.repeat_interleave(num_return_sequences, dim=0) for k, v in s.items()}
                                  for s in initial_states]
            B *= num_return_sequences
        dev = input_ids.device
        V = self.config.vocab_size

        logits, states = self.forward_with_state(input_ids, initial_states, last_only=True)
        nxt = logits[:, -1, :].float()
        use_pen = repetition_penalty is not None and repetition_penalty != 1.0 and repetition_penalty > 0
        seen = None
        if use_pen:
            seen = torch.zeros(B, V, dtype=torch.bool, device=dev)
            seen.scatter_(1, input_ids.clamp(0, V - 1), True)
        ban = torch.tensor(token_ban, dtype=torch.long, device=dev) if token_ban else None
        eos_t = torch.tensor(eos_ids, dtype=torch.long, device=dev) if eos_ids else None
        unfinished = torch.ones(B, dtype=torch.bool, device=dev)
        pieces = [input_ids]
        for _ in range(max(budget, 0)):
            if use_pen:
                apply_repetition_penalty_(nxt, seen, repetition_penalty)
            if ban is not None:
                nxt[:, ban] = float("-inf")
            tok = sample_from_logits(nxt, do_sample, temperature, top_k, top_p if do_sample else 0.0, generator)
            pieces.append(tok.unsqueeze(1))
            if use_pen:
                seen.scatter_(1, tok.unsqueeze(1), True)
            if eos_t is not None:
                unfinished &= ~torch.isin(tok, eos_t)
                if not bool(unfinished.any()):
                    break
            logits, states = self.forward_with_state(tok.unsqueeze(1), states, last_only=True)
            nxt = logits[:, -1, :].float()
        out = torch.cat(pieces, dim=1)
        if return_dict_in_generate:
            return {"sequences": out, "states": states}
        return out
