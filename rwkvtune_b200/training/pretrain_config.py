"""``PretrainConfig`` (``rwkvtune/training/pretrain_config.py:47-116``): the SFT record with the
pre-training defaults ``weight_decay=0.01``, ``epoch_save=5``, ``proj_dir="output_pretrain"``."""
from __future__ import annotations

from dataclasses import dataclass

from .sft_config import SFTConfig


@dataclass
class PretrainConfig(SFTConfig):
    weight_decay: float = 0.01
    epoch_save: int = 5
    proj_dir: str = "output_pretrain"
