"""GRPO-family objectives (``rwkvtune/training/grpo/loss.py:14-213``).

Per token: ``ratio = exp(logp - logp_old)`` (token level) or the sequence mean of the log-ratio
(GSPO), PPO clipping to ``[1 - eps, 1 + eps_high]``, ``-min(r A, clip(r) A)``, plus
``beta * (exp(ref - logp) - (ref - logp) - 1)``, times the completion mask.  Aggregation: ``dapo`` /
``grpo`` sum over mask count, ``dr_grpo`` sum over ``N * max_completion_length``, ``bnpo`` local count.
"""
from __future__ import annotations

from typing import Optional

import torch


class GRPOLossBase:
    def __init__(self, epsilon: float = 0.2, epsilon_high: Optional[float] = None, delta: Optional[float] = None,
                 importance_sampling_level: str = "token"):
        if importance_sampling_level not in ("token", "sequence"):
            raise ValueError("importance_sampling_level must be 'token' or 'sequence'")
        self.epsilon = epsilon
        self.epsilon_high = epsilon if epsilon_high is None else epsilon_high
        self.delta = delta
        self.importance_sampling_level = importance_sampling_level

    def compute_loss(self, per_token_loss: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def importance_ratio(self, logps_policy, logps_sampling, mask):
        log_ratio = logps_policy - logps_sampling
        if self.importance_sampling_level == "sequence":
            log_ratio = ((log_ratio * mask).sum(-1) / mask.sum(-1).clamp(min=1.0)).unsqueeze(-1)
        return torch.exp(log_ratio)

    def compute_per_token_loss(self, logps_policy, logps_ref, logps_sampling, advantages, mask, beta: float = 0.0):
        ratio = self.importance_ratio(logps_policy, logps_sampling, mask)
        adv = advantages.unsqueeze(1)
        clipped = torch.clamp(ratio, 1.0 - self.epsilon, 1.0 + self.epsilon_high)
        loss = -torch.min(ratio * adv, clipped * adv)
        if beta > 0.0 and logps_ref is not None:
            d = logps_ref - logps_policy
            loss = loss + beta * (torch.exp(d) - d - 1)
        return loss * mask


class DAPOLoss(GRPOLossBase):
    def compute_loss(self, per_token_loss, mask):
        return (per_token_loss * mask).sum() / mask.sum().clamp(min=1.0)


class DrGRPOLoss(GRPOLossBase):
    def __init__(self, max_completion_length: int, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.max_completion_length = max_completion_length

    def compute_loss(self, per_token_loss, mask):
        return (per_token_loss * mask).sum() / (per_token_loss.shape[0] * self.max_completion_length)


class BNPOLoss(GRPOLossBase):
    def compute_loss(self, per_token_loss, mask):
        return (per_token_loss * mask).sum() / mask.sum().clamp(min=1.0)


def get_loss_function(loss_type: str, config) -> GRPOLossBase:
    kw = dict(epsilon=config.epsilon, epsilon_high=config.epsilon_high, delta=config.delta,
              importance_sampling_level=config.importance_sampling_level)
    if loss_type in ("dapo", "grpo"):
        return DAPOLoss(**kw)
    if loss_type == "dr_grpo":
        return DrGRPOLoss(config.max_completion_length, **kw)
    if loss_type == "bnpo":
        return BNPOLoss(**kw)
    raise ValueError(f"unknown loss type {loss_type!r}; available: dapo, dr_grpo, bnpo, grpo")
