"""Log-probability helpers (``rwkvtune/training/grpo/utils.py:13-152``).

The functions that take *logits* are kept for API parity and small inputs; the trainer itself never
materialises ``[n, L, V]`` logits but calls :func:`rwkvtune_b200.ops.linear_logprob_entropy` on the
hidden states, which fuses the vocabulary head with the gather / log-sum-exp / entropy.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[..., index]`` computed row by row so that no full log-softmax copy exists."""
    out = torch.empty(index.shape, dtype=torch.float32, device=logits.device)
    flat_logits = logits.reshape(-1, logits.shape[-2], logits.shape[-1]) if logits.dim() > 2 else logits.unsqueeze(0)
    flat_index = index.reshape(flat_logits.shape[0], -1)
    flat_out = out.view(flat_logits.shape[0], -1)
    for i in range(flat_logits.shape[0]):
        row = flat_logits[i].float()
        flat_out[i] = row.gather(-1, flat_index[i].unsqueeze(-1)).squeeze(-1) - torch.logsumexp(row, dim=-1)
    return out


def entropy_from_logits(logits: torch.Tensor, chunk_size: int = 128) -> torch.Tensor:
    flat = logits.reshape(-1, logits.shape[-1])
    outs = []
    for c in flat.split(chunk_size, dim=0):
        lp = F.log_softmax(c.float(), dim=-1)
        outs.append(-(lp.exp() * lp).sum(-1))
    return torch.cat(outs).reshape(logits.shape[:-1])
