"""User callbacks of the trainers.

In the reference the work around each micro-batch (learning-rate schedule, loss all-reduce, throughput
and loss logs, checkpoint rotation) lives in a Lightning callback (``rwkvtune/training/callbacks.py:20-512``,
``TrainingCallback``; ``rwkvtune/training/grpo_trainer.py:34-259``, ``GRPOTrainingCallback``), and
``GRPOTrainer(callbacks=[...])`` hands further Lightning callbacks to ``lightning.Trainer``
(``grpo_trainer.py:311-324``, ``:720-745``).  Here that fixed work is part of the trainers and of
``engine/metrics.py``; this module keeps the extension point.  A callback is any object with some of the
hooks below; ``SFTTrainer`` / ``PretrainTrainer`` / ``GRPOTrainer`` take ``callbacks=[...]`` and call them on
every rank:

================================  =====================================================================
``on_train_start(trainer)``       engine built, resume done, before the first batch
``on_train_batch_start(trainer,   before a micro-batch is stepped (``batch`` is the host batch dict)
batch, batch_idx)``
``on_train_batch_end(trainer,     after it; ``outputs`` is ``{"loss": float, "lr": float, ...}`` (GRPO adds
outputs, batch, batch_idx)``      its clip, KL, entropy and reward statistics)
``on_step_end(trainer, metrics)`` same moment, metrics only (the form the GRPO trainer always offered)
``on_train_epoch_end(trainer,     after the last batch of an epoch, before the epoch's save point
epoch)``
``on_save_checkpoint(trainer,     after a save point has been published (every rank; files are written by
path)``                           rank 0)
``on_train_end(trainer)``         after the last save point
================================  =====================================================================

Callbacks written against Lightning's signatures (``hook(trainer, pl_module, ...)``) are called with the
model in the ``pl_module`` position, so a callback that only reads ``pl_module.parameters()`` or the batch
works unchanged; anything that reaches into ``lightning.Trainer`` internals does not.
"""
from __future__ import annotations

import inspect
from typing import Any, Iterable, List


class TrainingCallback:
    """Base class with every hook as a no-op; subclass and override what is needed."""

    def on_train_start(self, trainer) -> None: ...
    def on_train_batch_start(self, trainer, batch, batch_idx: int) -> None: ...
    def on_train_batch_end(self, trainer, outputs, batch, batch_idx: int) -> None: ...
    def on_step_end(self, trainer, metrics) -> None: ...
    def on_train_epoch_end(self, trainer, epoch: int) -> None: ...
    def on_save_checkpoint(self, trainer, path: str) -> None: ...
    def on_train_end(self, trainer) -> None: ...


_MODULE_ARG_NAMES = ("pl_module", "module", "lightning_module")


def _wants_module(fn) -> bool:
    """True when the hook's second parameter is Lightning's module argument."""
    try:
        params = [p for p in inspect.signature(fn).parameters.values()
                  if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    except (TypeError, ValueError):
        return False
    return len(params) >= 2 and params[1].name in _MODULE_ARG_NAMES


class CallbackList:
    """Holds the user's callbacks and calls one hook on all of them, in order."""

    def __init__(self, callbacks: Iterable[Any] = ()):
        self.callbacks: List[Any] = list(callbacks or [])

    def __iter__(self):
        return iter(self.callbacks)

    def __len__(self) -> int:
        return len(self.callbacks)

    def append(self, cb) -> None:
        self.callbacks.append(cb)

    def fire(self, hook: str, trainer, *args) -> None:
        for cb in self.callbacks:
            fn = getattr(cb, hook, None)
            if fn is None:
                continue
            if _wants_module(fn):
                fn(trainer, getattr(trainer, "model", None), *args)
            else:
                fn(trainer, *args)
