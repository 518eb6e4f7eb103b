"""Shared implementation of ``SFTTrainer`` and ``PretrainTrainer``.

The reference builds a ``lightning.Trainer`` around a LightningModule and a callback
(``rwkvtune/training/sft_trainer.py:90-817``, ``pretrain_trainer.py:63-578``,
``callbacks.py:123-502``).  Here the trainer drives :class:`TrainEngine` directly: one process per
GPU (adopted from the launcher environment, or spawned when ``devices > 1`` and no launcher is
present), a per-rank :class:`BatchLoader`, the micro-batch learning-rate schedule, metric sinks,
atomic checkpoints with rotation, and resume by seeking the sampler.
"""
from __future__ import annotations

import copy
import dataclasses
import os
import time
from typing import Any, Dict, Optional

import torch

from ..engine import EngineConfig, TrainEngine, sft_lr
from ..engine import checkpoint as ckpt
from ..engine.metrics import MetricLogger
from ..models import AutoModel
from ..parallel import init_distributed
from ..peft import LoraConfig, get_peft_model, is_peft_model
from .callbacks import CallbackList
from .data_loading import BatchLoader
from .model_save_utils import save_model_or_adapter

_ARCH_FIELDS = ("n_layer", "n_embd", "vocab_size", "head_size_a", "dim_att_lora", "dim_gate_lora", "dim_mv_lora",
                "dim_att", "dim_ffn")


def _spawn_entry(local_rank: int, trainer, port: int):
    os.environ.update({"RANK": str(local_rank), "LOCAL_RANK": str(local_rank), "WORLD_SIZE": str(trainer.args.devices),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    trainer._train_worker()


class SupervisedTrainer:
    config_name = "sft"
    accepts_iterable = False

    def __init__(self, model, args, train_dataset, processing_class=None, lora_config: Optional[LoraConfig] = None,
                 callbacks=None):
        self.args = args
        self.callbacks = CallbackList(callbacks)
        self.train_dataset = train_dataset
        self.processing_class = processing_class
        self.lora_config = lora_config
        self.base_model_path = model if isinstance(model, str) else ""
        self._validate_dataset(train_dataset)
        if isinstance(model, str):
            model = AutoModel.from_pretrained(model, device="cpu")
        self.model = model
        if lora_config is not None and not is_peft_model(model):
            if isinstance(lora_config, dict):   # the reference passes the adapter settings as a plain dict
                known = {f.name for f in dataclasses.fields(LoraConfig)}
                lora_config = LoraConfig(**{k: v for k, v in lora_config.items() if k in known})
            self.model = get_peft_model(model, lora_config)
        args.use_lora = is_peft_model(self.model)
        self._sync_arch_fields()
        self.engine: Optional[TrainEngine] = None
        self.ctx = None
        self.state: Dict[str, Any] = {"samples_seen": 0, "epoch": 0, "global_batch": 0}

    # ------------------------------------------------------------------ set-up
    def _validate_dataset(self, ds) -> None:
        if ds is None:
            raise ValueError("train_dataset is required")
        iterable = not (hasattr(ds, "__getitem__") and hasattr(ds, "__len__"))
        if iterable:
            if not self.accepts_iterable:
                raise TypeError(f"{type(self).__name__} needs a map-style dataset with input_ids and labels")
            return
        if len(ds) == 0:
            raise ValueError("train_dataset is empty")
        cols = getattr(ds, "column_names", None)
        first = ds[0]
        keys = set(cols) if cols else set(first.keys())
        missing = {"input_ids", "labels"} - keys
        if missing:
            raise ValueError(f"train_dataset lacks columns {sorted(missing)}; samples must carry pre-shifted "
                             "'input_ids' and 'labels' (labels[i] is the target of position i, -100 = ignore)")

    def _sync_arch_fields(self) -> None:
        mc = self.model.config
        for f in _ARCH_FIELDS:
            if hasattr(mc, f):
                setattr(self.args, f, getattr(mc, f))
        mc.grad_cp = self.args.grad_cp
        mc.ctx_len = self.args.ctx_len

    def _engine_config(self) -> EngineConfig:
        a = self.args
        return EngineConfig(lr_init=a.lr_init, beta1=a.beta1, beta2=a.beta2, adam_eps=a.adam_eps,
                            weight_decay=a.weight_decay, grad_clip=a.grad_clip,
                            accumulate_grad_batches=a.accumulate_grad_batches, strategy=a.strategy,
                            precision=a.precision if a.accelerator != "cpu" else "fp32", grad_cp=a.grad_cp,
                            lr_2x_patterns=("att.w0",) if a.train_type == "infctx" else (),
                            train_type=a.train_type, chunk_ctx=a.chunk_ctx, truncated_bptt=a.truncated_bptt,
                            transport=os.environ.get("RWKVTUNE_TRANSPORT", "auto"),
                           cuda_graph=os.environ.get("RWKVTUNE_CUDA_GRAPH", "0") == "1")

    # ------------------------------------------------------------------ public
    def train(self) -> None:
        a = self.args
        launched = int(os.environ.get("WORLD_SIZE", "1")) > 1
        if a.devices > 1 and not launched and a.accelerator != "cpu":
            import torch.multiprocessing as mp

            port = 29500 + (os.getpid() % 2000)
            mp.start_processes(_spawn_entry, args=(self, port), nprocs=a.devices, join=True, start_method="spawn")
            return
        self._train_worker()

    def save_model(self, output_dir: Optional[str] = None) -> str:
        out = output_dir or os.path.join(self.args.proj_dir, "final")
        if self.ctx is None or self.ctx.is_main:
            save_model_or_adapter(self.model, out, self.processing_class, self.args.lora_save_mode,
                                              self.base_model_path)
        return out

    # ------------------------------------------------------------------ worker
    def _train_worker(self) -> None:
        a = self.args
        ctx = self.ctx = init_distributed("cpu" if a.accelerator == "cpu" else "gpu")
        if a.seed >= 0:
            torch.manual_seed(a.seed)
        if a.train_type == "infctx" and a.accumulate_grad_batches > 1 and self.config_name == "pretrain":
            raise ValueError("accumulate_grad_batches > 1 is not supported for infctx pre-training")
        self.engine = eng = TrainEngine(self.model, self._engine_config(), ctx)
        self.model = eng.model
        loader = BatchLoader(self.train_dataset, a.micro_bsz, a.ctx_len, ctx.rank, ctx.world_size,
                             a.dataloader_shuffle, max(a.seed, 0), pin=ctx.device.type == "cuda")
        per_epoch = loader.batches_per_epoch()
        if a.epoch_steps is not None:
            limit = max(1, a.epoch_steps // max(ctx.world_size, 1))
            per_epoch = limit if per_epoch is None else min(per_epoch, limit)
        if per_epoch is None:
            raise ValueError("an iterable dataset needs epoch_steps")
        if per_epoch == 0:
            raise ValueError("dataset too small for one batch per rank (micro_bsz x devices samples needed)")
        total_steps = per_epoch * a.epoch_count
        logger = MetricLogger(a.proj_dir, a.report_to, a.run_name, ctx.is_main, config=vars(a))
        start_epoch, skip = self._maybe_resume(per_epoch)
        samples_per_batch = a.micro_bsz * ctx.world_size
        guard = eng.start_guard()
        self.callbacks.fire("on_train_start", self)
        try:
            self._run_epochs(start_epoch, skip, per_epoch, total_steps, loader, logger, samples_per_batch)
        except Exception as exc:
            self._emergency_save(exc)
            raise
        finally:
            if guard is not None:
                guard.stop()
        self.callbacks.fire("on_train_end", self)
        logger.close()
        ctx.barrier()

    def _run_epochs(self, start_epoch, skip, per_epoch, total_steps, loader, logger, samples_per_batch) -> None:
        from ..engine.profiling import StepProfiler, profile_steps_requested

        a, ctx, eng = self.args, self.ctx, self.engine
        profiler = StepProfiler(profile_steps_requested(a), a.proj_dir, is_main=ctx.is_main)
        tuned = False
        for epoch in range(start_epoch, a.epoch_count):
            self.state["epoch"] = epoch
            loss_sum, n_loss = 0.0, 0
            t_last = time.perf_counter()
            for b, batch in enumerate(loader.iter_epoch(epoch, skip), start=skip):
                if b >= per_epoch:
                    break
                real_step = (epoch + a.epoch_begin) * per_epoch + (b + 1)
                lr = sft_lr(real_step, a.lr_init, a.lr_final, a.warmup_steps, total_steps, a.epoch_count)
                self.callbacks.fire("on_train_batch_start", self, batch, b)
                profiler.step_begin()
                loss = eng.train_step_from_host(batch["input_ids"], batch["labels"], lr)
                profiler.step_end()
                self.state["samples_seen"] += samples_per_batch
                self.state["global_batch"] += 1
                if not tuned:
                    tuned = True
                    self._tune_checkpointing(batch["input_ids"].shape[1])
                if ctx.world_size > 1 and (b + 1) % a.log_every_n_steps == 0:
                    t = torch.tensor([loss], device=ctx.device)
                    torch.distributed.all_reduce(t)
                    loss = float(t) / ctx.world_size
                loss_sum += loss
                n_loss += 1
                now = time.perf_counter()
                if (b + 1) % a.log_every_n_steps == 0:
                    tokens = batch["input_ids"].numel() * ctx.world_size
                    rec = logger.log_step(self.state["global_batch"], loss, lr, tokens, now - t_last,
                                          eng.phases.scalars())
                    if ctx.is_main:
                        print(f"epoch {epoch} step {b + 1}/{per_epoch} loss {loss:.4f} lr {lr:.3e} "
                              f"{rec['kt_s']:.1f} Kt/s", flush=True)
                t_last = now
                if len(self.callbacks):
                    outputs = {"loss": loss, "lr": lr}
                    self.callbacks.fire("on_train_batch_end", self, outputs, batch, b)
                    self.callbacks.fire("on_step_end", self, outputs)
                if a.save_every_n_batches > 0 and self.state["global_batch"] % a.save_every_n_batches == 0:
                    self._save_checkpoint(f"rwkv7-batch{self.state['global_batch']}")
            skip = 0
            logger.log_epoch(epoch, loss_sum / max(n_loss, 1), self.state["global_batch"])
            self.callbacks.fire("on_train_epoch_end", self, epoch)
            if (a.epoch_save > 0 and (epoch + 1) % a.epoch_save == 0) or epoch == a.epoch_count - 1:
                self._save_checkpoint(f"rwkv7-epoch{epoch + 1}")

    def _tune_checkpointing(self, first_len: int) -> None:
        """After the first step (every block recomputed, memory peak known): keep the activations of as many blocks as
        fit and recompute only the rest (``TrainEngine.autotune_checkpointing``).  Only for ``grad_cp=1`` in normal mode
        on a GPU, and only when the first batch of every rank was ``ctx_len`` long - with shorter first batches the
        measured peak says nothing about the longest one, and every block stays recomputed as in the reference.
        ``RWKVTUNE_GRAD_CP_AUTO=0`` switches it off."""
        a, ctx, eng = self.args, self.ctx, self.engine
        if not a.grad_cp or a.train_type != "normal" or ctx.device.type != "cuda":
            return
        if os.environ.get("RWKVTUNE_GRAD_CP_AUTO", "1") == "0":
            return
        full = ctx.all_agree(first_len >= a.ctx_len)          # one host-side agreement: every rank takes the same branch
        if not full:
            return
        n_cp = eng.autotune_checkpointing(a.micro_bsz, a.ctx_len)
        if ctx.is_main:
            print(f"activation checkpointing: {n_cp} of {eng.model.config.n_layer} blocks recomputed", flush=True)

    def _emergency_save(self, exc: BaseException) -> None:
        """A peer stopped answering or a step was aborted: the lowest rank still known to be alive writes a
        weights-only save point without any collective (the reference has no counterpart; its elastic resume reloads
        weights only, ``rwkvtune/training/sft_trainer.py:705-723``).  Parameters are consistent: an aborted step's
        kernels leave them untouched."""
        from ..engine.watchdog import RankFailure, StepAborted
        from ..parallel.p2p import PeerWaitTimeout

        if not isinstance(exc, (RankFailure, StepAborted, PeerWaitTimeout)) or self.ctx is None:
            return
        dead = set(exc.ranks) if isinstance(exc, RankFailure) else set()
        writer = min(r for r in range(self.ctx.world_size) if r not in dead)
        if self.ctx.rank != writer:
            return
        out = os.path.join(self.args.proj_dir, "rwkv7-emergency")
        try:
            save_model_or_adapter(self.model, out, self.processing_class, self.args.lora_save_mode, self.base_model_path)
            with open(os.path.join(out, "emergency.txt"), "w", encoding="utf-8") as fh:
                fh.write(f"{type(exc).__name__}: {exc}\nsamples_seen={self.state['samples_seen']}\n")
            print(f"[trainer] {type(exc).__name__}: weights saved to {out}", flush=True)
        except Exception as save_exc:   # never mask the original failure
            print(f"[trainer] emergency save failed: {save_exc}", flush=True)

    # ------------------------------------------------------------------ checkpoints
    def _save_checkpoint(self, name: str) -> None:
        a, ctx, eng = self.args, self.ctx, self.engine
        eng.check_health()    # never write a save point from a step in which a device-side wait expired
        final = os.path.join(a.proj_dir, name)
        meta = {"samples_seen": self.state["samples_seen"], "devices": ctx.world_size, "micro_bsz": a.micro_bsz,
                "accumulate_grad_batches": a.accumulate_grad_batches, "epoch": self.state["epoch"],
                "global_batch": self.state["global_batch"], "trainer": self.config_name}

        def write(tmp: str) -> None:
            if ctx.is_main:
                save_model_or_adapter(self.model, tmp, self.processing_class, a.lora_save_mode,
                                                  self.base_model_path)
            ckpt.save_trainer_state(tmp, eng, ctx, meta, a.save_optimizer_state)

        ckpt.atomic_checkpoint(final, ctx, write)
        if ctx.is_main and a.save_total_limit > 0:
            ckpt.rotate_checkpoints(a.proj_dir, a.save_total_limit)
        ctx.barrier()
        self.callbacks.fire("on_save_checkpoint", self, final)

    def _maybe_resume(self, per_epoch: int):
        a, ctx, eng = self.args, self.ctx, self.engine
        path = a.resume_from_checkpoint
        if not path:
            return 0, 0
        if path == "latest":
            path = a.proj_dir
        found = ckpt.find_checkpoint(path)
        if found is None:
            raise FileNotFoundError(f"no checkpoint found at {a.resume_from_checkpoint}")
        self._load_weights(found)
        meta = ckpt.read_meta(found) if os.path.isdir(found) else {}
        restored = ckpt.load_optimizer_state(found, eng, ctx) if os.path.isdir(found) else False
        if not restored:
            eng.opt.master.copy_(eng.space.params[eng.opt.lo:eng.opt.hi].float())
        samples = int(meta.get("samples_seen", 0))
        self.state["samples_seen"] = samples
        batches_done = samples // (a.micro_bsz * ctx.world_size)
        self.state["global_batch"] = batches_done
        if ctx.is_main:
            mode = "with optimizer state" if restored else "weights only"
            print(f"resumed from {found} ({mode}); samples_seen={samples}, saved world={meta.get('devices')}, "
                  f"current world={ctx.world_size}")
        return batches_done // per_epoch, batches_done % per_epoch

    def _load_weights(self, found: str) -> None:
        from ..models.auto_model import load_weight_file

        model = self.model
        if os.path.isdir(found):
            adapter = os.path.join(found, "adapter_model.bin")
            full = next((os.path.join(found, n) for n in ("model.pth", "model.safetensors")
                         if os.path.exists(os.path.join(found, n))), None)
            if is_peft_model(model) and os.path.exists(adapter):
                model.load_lora_weights(adapter)
                return
            if full is None:
                raise FileNotFoundError(f"{found} has neither model weights nor adapter weights")
            sd = load_weight_file(full)
        else:
            if found.endswith("adapter_model.bin") and is_peft_model(model):
                model.load_lora_weights(found)
                return
            sd = load_weight_file(found)
        if is_peft_model(model):
            own = model.state_dict()
            alias = {k.replace(".base_layer.", "."): k for k in own}
            sd = {alias.get(k, k): v for k, v in sd.items()}
        with torch.no_grad():
            own = model.state_dict()
            for k, v in sd.items():
                if k in own and own[k].shape == v.shape:
                    own[k].copy_(v.to(own[k].dtype))
