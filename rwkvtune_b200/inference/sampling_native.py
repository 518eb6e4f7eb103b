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
