"""Infinite-context view of the model: logits for one chunk plus the state to hand to the next.

The reference keeps a second copy of every layer class for this
(``rwkvtune/models/rwkv7/model_infctx.py:17-255``).  Here the ordinary blocks already
take and return state, so ``RWKV7Infctx`` is the same module with the
``forward_infctx`` calling convention; parameter names are unchanged and the two
classes share a ``state_dict``.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .model import RWKV7Model


class RWKV7Infctx(RWKV7Model):
    def forward_hidden_infctx(self, idx: torch.Tensor, shift_states: torch.Tensor, wkv_states: torch.Tensor,
                              checkpoint: bool = False):
        L = self.config.n_layer
        att_prev = [shift_states[i, 0] for i in range(L)]
        ffn_prev = [shift_states[i, 1] for i in range(L)]
        wkv = [wkv_states[i] for i in range(L)]
        x, a_l, s_l, f_l = self.forward_states(idx, att_prev, wkv, ffn_prev, checkpoint=checkpoint)
        new_shift = torch.stack([torch.stack([a, f], dim=0) for a, f in zip(a_l, f_l)], dim=0)
        new_wkv = torch.stack(s_l, dim=0)
        return x, new_shift, new_wkv

    def forward_infctx(self, idx: torch.Tensor, last_shift_states: torch.Tensor, last_wkv_states: torch.Tensor
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``idx [B, T]``, ``shift_states [L,2,B,C]``, ``wkv_states [L,B,H,N,N]`` ->
        ``(logits [B,T,V], new_shift_states, new_wkv_states)``."""
        x, new_shift, new_wkv = self.forward_hidden_infctx(idx, last_shift_states, last_wkv_states)
        return self.head(x), new_shift, new_wkv


def as_infctx(model: RWKV7Model) -> RWKV7Infctx:
    """Re-class an existing model in place (no parameter copy)."""
    if not isinstance(model, RWKV7Infctx):
        model.__class__ = RWKV7Infctx
    return model
