"""Trainers (public names of ``rwkvtune/training/__init__.py:26-41``)."""
from .pretrain_config import PretrainConfig
from .pretrain_trainer import PretrainTrainer
from .sft_config import SFTConfig
from .sft_trainer import SFTTrainer

from ..ops.reference import L2Wrap

__all__ = ["PretrainConfig", "PretrainTrainer", "SFTConfig", "SFTTrainer", "GRPOConfig", "GRPOTrainer", "L2Wrap"]


def __getattr__(name):
    if name in ("GRPOConfig", "GRPOTrainer"):
        from . import grpo_config, grpo_trainer

        return {"GRPOConfig": grpo_config.GRPOConfig, "GRPOTrainer": grpo_trainer.GRPOTrainer}[name]
    raise AttributeError(name)
