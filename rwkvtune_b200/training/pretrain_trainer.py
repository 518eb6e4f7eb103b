"""``PretrainTrainer`` (``rwkvtune/training/pretrain_trainer.py:63-578``).

Accepts map-style and iterable datasets.  Unlike the reference, which builds a fresh randomly
initialised network and ignores the weights of the model it was handed
(``pretrain_trainer.py:151-178``), this trainer trains the model it is given.
``resume_from_checkpoint="latest"`` picks the newest checkpoint under ``proj_dir``.
"""
from __future__ import annotations

from .pretrain_config import PretrainConfig
from .trainer_base import SupervisedTrainer


class PretrainTrainer(SupervisedTrainer):
    config_name = "pretrain"
    accepts_iterable = True

    def __init__(self, model, args: PretrainConfig = None, train_dataset=None, processing_class=None, lora_config=None,
                 callbacks=None):
        super().__init__(model, args or PretrainConfig(), train_dataset, processing_class, lora_config, callbacks)
