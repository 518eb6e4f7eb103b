"""``SFTTrainer`` (``rwkvtune/training/sft_trainer.py:90-817``): supervised fine-tuning on a dataset of
pre-shifted ``input_ids`` / ``labels``; optional LoRA; standard or infinite-context mode."""
from __future__ import annotations

from .sft_config import SFTConfig
from .trainer_base import SupervisedTrainer


class SFTTrainer(SupervisedTrainer):
    config_name = "sft"
    accepts_iterable = False

    def __init__(self, model, args: SFTConfig = None, train_dataset=None, processing_class=None, lora_config=None,
                 callbacks=None):
        super().__init__(model, args or SFTConfig(), train_dataset, processing_class, lora_config, callbacks)
