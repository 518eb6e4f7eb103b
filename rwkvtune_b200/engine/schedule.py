"""Learning-rate schedules of the three trainers.

``sft_lr`` is the per-micro-batch warm-up + cosine rule of ``rwkvtune/training/callbacks.py:123-152``;
``grpo_lr_scale`` is the LambdaLR rule of ``rwkvtune/training/grpo/lightning_module.py:2098-2121``
(stepped once per optimiser step, progress measured in training steps).
"""
from __future__ import annotations

import math


def sft_lr(real_step: int, lr_init: float, lr_final: float, warmup_steps: int, total_steps: int,
           epoch_count: int = 1) -> float:
    if warmup_steps > 0 and real_step < warmup_steps:
        return lr_init * real_step / warmup_steps
    if lr_final == lr_init or epoch_count == 0 or warmup_steps >= total_steps:
        return lr_init
    progress = (real_step - warmup_steps) / max(1, total_steps - warmup_steps)
    progress = min(max(progress, 0.0), 1.0)
    return lr_final + (lr_init - lr_final) * (0.5 + 0.5 * math.cos(math.pi * progress))


def grpo_lr_scale(optimizer_step: int, lr_init: float, lr_final: float, warmup_steps: int,
                  total_optimizer_steps: int, accumulate: int) -> float:
    actual = optimizer_step * accumulate
    if actual < warmup_steps:
        return actual / max(1, warmup_steps)
    total = total_optimizer_steps * accumulate
    if warmup_steps >= total:
        return 1.0
    progress = min((actual - warmup_steps) / max(1, total - warmup_steps), 1.0)
    cosine = 0.5 * (1.0 + math.cos(progress * math.pi))
    return lr_final / lr_init + (1.0 - lr_final / lr_init) * cosine
