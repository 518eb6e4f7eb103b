"""Metric sinks: console, ``loss_data.jsonl``, ``train_log.txt``, TensorBoard, SwanLab / W&B when present.

File names, record keys and metric names follow ``rwkvtune/training/callbacks.py:113-295``.  Only
rank 0 writes.  Throughput counts the tokens actually processed (the reference assumes every sample
is ``ctx_len`` long); step time is the host wall-clock between two loss read-backs, each of which waits for
the step's kernels, so it includes device time and host time of the step.
"""
from __future__ import annotations

import datetime
import json
import math
import os
import time
from typing import Any, Dict, Optional


class MetricLogger:
    def __init__(self, proj_dir: str, report_to: str = "", run_name: str = "", is_main: bool = True,
                 loss_file: str = "loss_data.jsonl", log_file: str = "train_log.txt", config: Optional[dict] = None):
        self.is_main = is_main
        self.proj_dir = proj_dir
        self.loss_path = os.path.join(proj_dir, loss_file)
        self.log_path = os.path.join(proj_dir, log_file)
        self.tb = None
        self.ext = None
        self._last = time.time()
        if not is_main:
            return
        os.makedirs(proj_dir, exist_ok=True)
        with open(self.log_path, "a", encoding="utf-8") as fh:
            fh.write(f"NEW RUN {datetime.datetime.now().isoformat()}\n{json.dumps(config or {}, default=str)}\n")
        if report_to == "tensorboard":
            try:
                from torch.utils.tensorboard import SummaryWriter

                self.tb = SummaryWriter(os.path.join(proj_dir, "tensorboard", run_name or "run"))
            except Exception as exc:
                print(f"[metrics] tensorboard unavailable: {exc}")
        elif report_to in ("swanlab", "wandb"):
            try:
                mod = __import__(report_to)
                mod.init(project=os.path.basename(os.path.normpath(proj_dir)), name=run_name or None, config=config)
                self.ext = mod
            except Exception as exc:
                print(f"[metrics] {report_to} unavailable: {exc}")

    def log_step(self, step: int, loss: float, lr: float, tokens: int, step_seconds: float,
                 extra: Optional[Dict[str, float]] = None) -> Dict[str, float]:
        kt_s = tokens / max(step_seconds, 1e-9) / 1000.0
        rec = {"loss": loss, "t_cost": step_seconds, "kt_s": kt_s}
        if not self.is_main:
            return rec
        with open(self.loss_path, "a", encoding="utf-8") as fh:
            fh.write(json.dumps(rec) + "\n")
        scalars = {"train/loss": loss, "train/lr": lr, "train/throughput_kt_s": kt_s}
        scalars.update(extra or {})
        self._emit(scalars, step)
        return rec

    def log_epoch(self, epoch: int, mean_loss: float, step: int) -> None:
        if not self.is_main:
            return
        ppl = math.exp(min(mean_loss, 50.0))
        with open(self.log_path, "a", encoding="utf-8") as fh:
            fh.write(f"{epoch} {mean_loss:.6f} {ppl:.4f} {datetime.datetime.now().isoformat()}\n")
        self._emit({"train/epoch_loss": mean_loss, "train/epoch_perplexity": ppl, "train/epoch": epoch}, step)

    def log_scalars(self, scalars: Dict[str, float], step: int) -> None:
        if self.is_main:
            self._emit(scalars, step)

    def _emit(self, scalars: Dict[str, Any], step: int) -> None:
        if self.tb is not None:
            for k, v in scalars.items():
                self.tb.add_scalar(k, v, step)
        if self.ext is not None:
            self.ext.log(dict(scalars), step=step)

    def close(self) -> None:
        if self.tb is not None:
            self.tb.close()
        if self.ext is not None and hasattr(self.ext, "finish"):
            self.ext.finish()
