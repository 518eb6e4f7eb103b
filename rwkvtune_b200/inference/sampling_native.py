"""Binding of the sm_100a sampling kernel (``rwkvtune_b200/csrc/sampling.cu``)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ops import _ext

_SEED_COUNTER = [0x1234567]


def available() -> bool:
    return _ext.available() and hasattr(_ext.lib(), "rwkv_sample_top_p")


def sample_top_p(logits: torch.Tensor, temperature: float, top_p: float, max_valid_token_id: Optional[int],
                 seed: Optional[int] = None, generator: Optional[torch.Generator] = None,
                 out_tokens: Optional[torch.Tensor] = None, out_logp: Optional[torch.Tensor] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Temperature + top-p draw per row of ``[n, V]`` logits (bf16 or fp32), ids above
    ``max_valid_token_id`` banned.  Row ``i`` uses the Philox stream ``(seed, i)``."""
    n, V = logits.shape
    x = logits if logits.is_contiguous() else logits.contiguous()
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    if seed is None:
        if generator is not None:
            seed = int(torch.randint(0, 2 ** 62, (1,), generator=generator, device=generator.device))
        else:
            _SEED_COUNTER[0] = (_SEED_COUNTER[0] * 6364136223846793005 + 1442695040888963407) % (2 ** 63)
            seed = _SEED_COUNTER[0] ^ int(torch.initial_seed() & 0xFFFFFFFF)
    tokens = out_tokens if out_tokens is not None else torch.empty(n, dtype=torch.long, device=x.device)
    logp = out_logp if out_logp is not None else torch.empty(n, dtype=torch.float32, device=x.device)
    n_valid = V if max_valid_token_id is None else min(V, max_valid_token_id + 1)
    _ext.call("rwkv_sample_top_p", _ext.ptr(x), _ext.i32(1 if x.dtype == torch.bfloat16 else 0), _ext.i32(n), _ext.i32(V),
              _ext.i32(n_valid), _ext.f32(1.0 / temperature), _ext.f32(top_p), _ext.i64(seed), _ext.ptr(tokens),
              _ext.ptr(logp), _ext.stream())
    return tokens, logp


_BIAS_CACHE = {}


def bias_vector(logit_bias, V: int, device) -> Optional[torch.Tensor]:
    """Dense fp32 ``[V]`` vector of a ``{token id: bias}`` mapping (clamped to +-100), cached per mapping content."""
    if not logit_bias:
        return None
    key = (tuple(sorted((int(k), float(v)) for k, v in logit_bias.items())), V, str(device))
    vec = _BIAS_CACHE.get(key)
    if vec is None:
        if len(_BIAS_CACHE) > 16:
            _BIAS_CACHE.clear()
        vec = torch.zeros(V, dtype=torch.float32)
        for tid, b in key[0]:
            if 0 <= tid < V:
                vec[tid] += min(100.0, max(-100.0, b))
        vec = _BIAS_CACHE[key] = vec.to(device)
    return vec


def full_available() -> bool:
    return _ext.available() and hasattr(_ext.lib(), "rwkv_sample_tokens")


def sample_tokens(logits: torch.Tensor, temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0,
                  logit_bias=None, max_valid_token_id: Optional[int] = None, seen: Optional[torch.Tensor] = None,
                  seen_rows: Optional[torch.Tensor] = None, repetition_penalty: float = 1.0, update_seen: bool = False,
                  seed: Optional[int] = None, generator: Optional[torch.Generator] = None
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The whole sampling rule in one launch: repetition penalty from the ``seen`` bitmap (bool / uint8 ``[rows, V]``,
    row ``seen_rows[i]`` for batch row ``i``), banned ids, temperature (``< 1e-6``: greedy), logit bias, top-k, top-p,
    the draw, the token's log-probability under the filtered distribution, and (``update_seen``) marking the drawn
    token in the bitmap."""
    n, V = logits.shape
    x = logits if logits.is_contiguous() else logits.contiguous()
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    greedy = temperature < 1e-6
    if seed is None:
        if generator is not None:
            seed = int(torch.randint(0, 2 ** 62, (1,), generator=generator, device=generator.device))
        else:
            _SEED_COUNTER[0] = (_SEED_COUNTER[0] * 6364136223846793005 + 1442695040888963407) % (2 ** 63)
            seed = _SEED_COUNTER[0] ^ int(torch.initial_seed() & 0xFFFFFFFF)
    tokens = torch.empty(n, dtype=torch.long, device=x.device)
    logp = torch.empty(n, dtype=torch.float32, device=x.device)
    n_valid = V if max_valid_token_id is None else min(V, max_valid_token_id + 1)
    bias = bias_vector(logit_bias, V, x.device)
    seen_u8 = None
    if seen is not None:
        if seen.dtype not in (torch.bool, torch.uint8) or not seen.is_contiguous() or seen.shape[-1] != V:
            raise ValueError("seen must be a contiguous bool / uint8 [rows, V] bitmap")
        seen_u8 = seen.view(torch.uint8) if seen.dtype == torch.bool else seen
    rows = None if seen_rows is None else seen_rows.to(torch.int64).contiguous()
    _ext.call("rwkv_sample_tokens", _ext.ptr(x), _ext.i32(1 if x.dtype == torch.bfloat16 else 0), _ext.i32(n), _ext.i32(V),
              _ext.i32(n_valid), _ext.f32(1.0 if greedy else 1.0 / temperature), _ext.f32(top_p), _ext.i32(int(top_k or 0)),
              _ext.i32(1 if greedy else 0), _ext.ptr(bias), _ext.ptr(seen_u8), _ext.ptr(rows),
              _ext.f32(float(repetition_penalty or 1.0)), _ext.i32(1 if (update_seen and seen_u8 is not None) else 0),
              _ext.i64(seed), _ext.ptr(tokens), _ext.ptr(logp), _ext.stream())
    return tokens, logp


def advance_available() -> bool:
    return _ext.available() and hasattr(_ext.lib(), "rwkv_rollout_advance")


def rollout_advance(tok: torch.Tensor, rows: torch.Tensor, finished: torch.Tensor, out_ids: torch.Tensor,
                    lengths: torch.Tensor, eos: Optional[torch.Tensor], step: int,
                    next_tok: Optional[torch.Tensor] = None) -> None:
    """One launch for the per-step bookkeeping of a lock-step rollout: ``out_ids[rows, step] = tok`` (0 for finished rows),
    ``lengths[rows] += live``, ``finished[rows] |= tok in eos or last step``, and ``next_tok[:] = tok`` (the static input
    of a captured decode step).  Replaces about a dozen indexing kernels per step."""
    _ext.call("rwkv_rollout_advance", _ext.ptr(tok), _ext.ptr(rows), _ext.ptr(finished), _ext.ptr(out_ids),
              _ext.ptr(lengths), _ext.ptr(eos), _ext.i32(0 if eos is None else eos.numel()), _ext.i32(step),
              _ext.i32(out_ids.shape[1]), _ext.i32(tok.numel()), _ext.ptr(next_tok), _ext.stream())
