from .engine import EngineConfig, TrainEngine, resolve_stage
from .schedule import grpo_lr_scale, sft_lr

__all__ = ["EngineConfig", "TrainEngine", "resolve_stage", "sft_lr", "grpo_lr_scale"]
