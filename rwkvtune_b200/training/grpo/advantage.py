"""Group-relative advantages (``rwkvtune/training/grpo/advantage.py:11-192``)."""
from __future__ import annotations

from typing import Dict, Optional

import torch


class AdvantageCalculator:
    def __init__(self, scale_rewards: str = "group", num_generations: int = 8, advantage_clip: Optional[float] = None,
                 low_reward_threshold: Optional[float] = None, low_reward_scale: float = 0.01):
        if scale_rewards not in ("group", "batch", "none"):
            raise ValueError(f"scale_rewards must be group, batch or none, got {scale_rewards!r}")
        self.scale_rewards, self.G = scale_rewards, num_generations
        self.advantage_clip = advantage_clip
        self.low_reward_threshold, self.low_reward_scale = low_reward_threshold, low_reward_scale

    def _matrix(self, rewards: torch.Tensor) -> torch.Tensor:
        if rewards.shape[0] % self.G:
            raise ValueError(f"rewards count ({rewards.shape[0]}) must be divisible by num_generations ({self.G})")
        return rewards.view(-1, self.G)

    def compute_advantages(self, rewards: torch.Tensor) -> torch.Tensor:
        if self.scale_rewards == "none":
            return rewards
        R = self._matrix(rewards)
        if self.scale_rewards == "group":
            adv = (R - R.mean(1, keepdim=True)) / R.std(1, keepdim=True, unbiased=False).clamp(min=1e-8)
            if self.advantage_clip is not None:
                adv = adv.clamp(-self.advantage_clip, self.advantage_clip)
            if self.low_reward_threshold is not None:
                low = R.max(1, keepdim=True).values < self.low_reward_threshold
                adv = torch.where(low.expand_as(adv), adv * self.low_reward_scale, adv)
        else:
            adv = (R - R.mean()) / R.std(unbiased=False).clamp(min=1e-8)
            if self.advantage_clip is not None:
                adv = adv.clamp(-self.advantage_clip, self.advantage_clip)
        return adv.reshape(-1)

    def compute_group_statistics(self, rewards: torch.Tensor) -> Dict[str, torch.Tensor]:
        R = self._matrix(rewards)
        return {"group_mean_rewards": R.mean(1), "group_std_rewards": R.std(1, unbiased=False),
                "global_mean_reward": rewards.mean(), "global_std_reward": rewards.std(unbiased=False)}
