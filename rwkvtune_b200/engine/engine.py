"""Training engine: owns the device copy of the model, the flat parameter space, the sharded
optimiser and one training step (forward, fused loss, backward, reduce, clip, AdamW, publish).

It replaces ``lightning.Trainer`` + the DeepSpeed/DDP strategy objects that the reference's
trainers construct (``rwkvtune/training/sft_trainer.py:369-485``) and the ``training_step`` bodies
of its Lightning modules (``rwkvtune/training/lightning_module.py:175-206``,
``rwkvtune/training/lightning_module_infctx.py:213-417``).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Sequence

import torch

from .. import ops
from ..models.rwkv7.model_infctx import as_infctx
from ..parallel.bootstrap import DistContext
from ..parallel.flat import FlatParamSpace, build_param_groups
from ..parallel.zero import ZeroOptimizer

STRATEGY_STAGE = {"auto": 0, "ddp": 0, "single": 0, "deepspeed_stage_1": 1, "deepspeed_stage_2": 2,
                  "deepspeed_stage_2_offload": 2, "deepspeed_stage_3": 3, "deepspeed_stage_3_offload": 3}


def resolve_stage(strategy: str) -> int:
    if strategy not in STRATEGY_STAGE:
        raise ValueError(f"unknown strategy {strategy!r}; expected one of {sorted(STRATEGY_STAGE)}")
    return STRATEGY_STAGE[strategy]


@dataclass
class EngineConfig:
    lr_init: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.99
    adam_eps: float = 1e-8
    weight_decay: float = 0.0
    grad_clip: float = 1.0
    accumulate_grad_batches: int = 1
    strategy: str = "auto"
    precision: str = "bf16"
    grad_cp: int = 0
    lr_2x_patterns: Sequence[str] = ()
    train_type: str = "normal"
    chunk_ctx: int = 512
    truncated_bptt: bool = True
    transport: str = "auto"   # "p2p": fused kernels over symmetric memory; "nccl": library collectives; "auto": p2p on multi-GPU CUDA when symmetric memory can be set up
    l2wrap: bool = True
    grad_cp_layers: Optional[object] = None   # None = all layers when grad_cp=1; int k = first k layers; "auto"
    cuda_graph: bool = False   # replay forward+backward of a micro-batch (or of one infctx chunk) from a CUDA graph


class TrainEngine:
    def __init__(self, model: torch.nn.Module, cfg: EngineConfig, ctx: DistContext):
        self.cfg, self.ctx = cfg, ctx
        dtype = {"bf16": torch.bfloat16, "fp16": torch.bfloat16, "fp32": torch.float32}[cfg.precision]
        if ctx.device.type == "cpu":
            dtype = torch.float32
        self.model = model.to(device=ctx.device, dtype=dtype)
        self.model.config.grad_cp = cfg.grad_cp
        if isinstance(cfg.grad_cp_layers, int):
            self.model.config.grad_cp_layers = cfg.grad_cp_layers
        if cfg.train_type == "infctx":
            as_infctx(self.model)
        self.model.train()
        stage = resolve_stage(cfg.strategy)
        self.zero3 = None
        if stage == 3 and ctx.world_size > 1 and ctx.device.type == "cuda" and dtype == torch.bfloat16:
            from ..parallel.zero3 import Zero3ShardedLinears

            # trainable matrices are sharded too when the fused peer-memory transport carries their gradients;
            # on the library transport they stay replicated with sharded optimiser state (stage-2 behaviour)
            self.zero3 = Zero3ShardedLinears(self.model, ctx, shard_trainable=cfg.transport in ("p2p", "auto"))
        groups = build_param_groups(self.model.named_parameters(), cfg.weight_decay, cfg.lr_2x_patterns)
        if not groups:
            raise RuntimeError("the model has no trainable parameters")
        allocator = None
        transport = cfg.transport
        p2p_capable = ctx.world_size > 1 and ctx.device.type == "cuda" and stage >= 1 and dtype == torch.bfloat16
        if transport == "p2p" and ctx.world_size > 1 and not p2p_capable:
            raise ValueError("transport 'p2p' needs CUDA, bf16 and a ZeRO stage >= 1")
        if transport in ("p2p", "auto") and p2p_capable:
            try:
                from ..parallel.p2p import symmetric_allocator

                allocator = symmetric_allocator()
                transport = "p2p"
            except Exception as exc:   # no symmetric memory on this system: library collectives do the same job
                if cfg.transport == "p2p":
                    raise
                if ctx.is_main:
                    print(f"[engine] symmetric memory unavailable ({exc}); using NCCL collectives")
                transport = "nccl"
        elif transport == "auto":
            transport = "nccl"
        self.transport = transport
        self.space = FlatParamSpace(groups, ctx.world_size, dtype, ctx.device, allocator)
        self.stage = stage
        self.opt = ZeroOptimizer(self.space, ctx, min(stage, 2), (cfg.beta1, cfg.beta2), cfg.adam_eps, cfg.grad_clip,
                                 transport)
        if self.zero3 is not None and self.zero3.trainable:
            if self.opt._p2p is None:
                raise RuntimeError("ZeRO-3 with trainable sharded matrices needs the fused peer-memory transport")
            self.zero3.attach(self.opt._p2p, cfg.weight_decay, (cfg.beta1, cfg.beta2), cfg.adam_eps, cfg.grad_clip)
        if self.zero3 is not None:
            n_cp = self.model.config.n_layer if cfg.grad_cp else 0
            if cfg.grad_cp and isinstance(cfg.grad_cp_layers, int):
                n_cp = cfg.grad_cp_layers
            self.zero3.recompute_below = n_cp
        self.micro_step = 0
        self.optimizer_steps = 0
        self.tokens_seen = 0
        self._graphs: Dict[tuple, dict] = {}
        self.guard = None
        from .profiling import PhaseMonitor

        # phase timers + NVTX ranges; RWKVTUNE_PHASE_SYNC=1 synchronises at phase boundaries (exact device time per phase)
        self.phases = PhaseMonitor(ctx.device, sync=os.environ.get("RWKVTUNE_PHASE_SYNC", "0") == "1")

    # ------------------------------------------------------------------ memory-aware checkpointing
    SAVED_UNITS_PER_LAYER = 37.0   # [tokens, n_embd] bf16 tensors a block keeps for backward without checkpointing

    def autotune_checkpointing(self, batch: int, seq_len: int, reserve_fraction: float = 0.10) -> int:
        """With ``grad_cp=1`` the reference recomputes every block in backward.  180 GB of HBM usually has
        room to keep the activations of most blocks instead; this picks how many blocks still need
        checkpointing.  Call it after one full-checkpointing step so the peak of that step is known.
        Returns the number of checkpointed layers (also stored in ``model.config.grad_cp_layers``)."""
        cfg = self.model.config
        L = cfg.n_layer
        if self.ctx.device.type != "cuda" or not self.cfg.grad_cp:
            return L
        total = torch.cuda.get_device_properties(self.ctx.device).total_memory
        peak = self.phases.peak_bytes()
        per_layer = self.SAVED_UNITS_PER_LAYER * batch * seq_len * cfg.n_embd * 2
        budget = total * (1.0 - reserve_fraction) - peak
        free_layers = int(max(0, budget) // per_layer)
        n_cp = max(0, L - free_layers)
        if self.ctx.world_size > 1:   # every rank must make the same choice
            t = torch.tensor([n_cp], device=self.ctx.device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            n_cp = int(t)
        cfg.grad_cp_layers = n_cp
        if self.zero3 is not None:
            self.zero3.recompute_below = n_cp
        return n_cp

    # ------------------------------------------------------------------ losses
    def _loss_normal(self, idx: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        return self.model.loss(idx, labels, l2wrap=self.cfg.l2wrap)

    def _step_infctx(self, idx: torch.Tensor, labels: torch.Tensor, scale: float) -> torch.Tensor:
        """Chunked back-propagation through time.  Truncated mode back-propagates each chunk and
        detaches the carried state; full mode keeps the graph and back-propagates once
        (``rwkvtune/training/lightning_module_infctx.py:213-417``)."""
        cfg, m = self.cfg, self.model
        B, T = idx.shape
        C, L = m.config.n_embd, m.config.n_layer
        H, N = m.config.dim_att // m.config.head_size_a, m.config.head_size_a
        chunk = cfg.chunk_ctx
        n_chunks = (T + chunk - 1) // chunk
        shift = torch.zeros(L, 2, B, C, device=idx.device, dtype=m.dtype)
        wkv = torch.zeros(L, B, H, N, N, device=idx.device, dtype=torch.float32)
        total = torch.zeros((), device=idx.device, dtype=torch.float32)
        pending = []
        # which chunks have a supervised token: one device-to-host read for the whole sequence, so the chunk loop
        # below never waits for the GPU and the host can run ahead of it.  A chunk without one (a masked prompt)
        # contributes neither cross-entropy nor L2Wrap, but the sum is still divided by the number of chunks
        # (rwkvtune/training/lightning_module_infctx.py:246-262, :349-365).
        pad = n_chunks * chunk - T
        lab_p = torch.nn.functional.pad(labels, (0, pad), value=-100) if pad else labels
        chunk_valid = (lab_p.reshape(B, n_chunks, chunk) != -100).any(dim=2).any(dim=0).tolist()
        use_graph = cfg.truncated_bptt and self._graph_ok() and T % chunk == 0 and all(chunk_valid)
        for i in range(n_chunks):
            ids_c, lab_c = idx[:, i * chunk:(i + 1) * chunk], labels[:, i * chunk:(i + 1) * chunk]
            if use_graph:
                loss_c, shift, wkv = self._graph_chunk(ids_c, lab_c, shift, wkv, scale / n_chunks)
                total += loss_c
                continue
            x, shift, wkv = m.forward_hidden_infctx(ids_c, shift, wkv, checkpoint=bool(cfg.grad_cp))
            Bc, Tc, _ = x.shape
            if not cfg.truncated_bptt and not chunk_valid[i]:
                continue      # full BPTT: the chunk only carries state (and its graph) forward
            loss_c = ops.linear_cross_entropy(x.reshape(Bc * Tc, C), m._head_weight(), lab_c.reshape(-1),
                                              l2wrap=cfg.l2wrap, l2wrap_tokens=Bc * Tc)
            if cfg.truncated_bptt:
                if chunk_valid[i]:
                    (loss_c * (scale / n_chunks)).backward()
                    total += loss_c.detach()
                shift, wkv = shift.detach(), wkv.detach()
            else:
                pending.append(loss_c)
        if not cfg.truncated_bptt:
            if not pending:       # nothing supervised in the whole sequence
                return total
            loss = torch.stack(pending).sum() / n_chunks
            (loss * scale).backward()
            return loss.detach()
        return total / n_chunks

    # ------------------------------------------------------------------ CUDA-graph replay of forward + backward
    GRAPH_WARMUP_STEPS = 2     # eager steps before a shape is captured (allocator, lazy module state)

    def _graph_ok(self) -> bool:
        return (self.cfg.cuda_graph and self.ctx.device.type == "cuda" and self.zero3 is None
                and self.optimizer_steps >= self.GRAPH_WARMUP_STEPS)

    def _capture(self, key: tuple, build) -> dict:
        """Records ``build()`` (forward, loss, backward on static tensors) into a CUDA graph.  Small batches are bound
        by host-side launch cost (a few thousand launches per step); a replay issues them in one call.  Parameter
        gradients accumulate into the flat gradient buffer exactly as in eager mode.  Cached fp32 parameter copies
        are invalidated first so that their refresh kernels are part of the recording."""
        ops.bump_param_epoch()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        entry = {"graph": torch.cuda.CUDAGraph()}
        from ..ops import _ext

        with torch.cuda.stream(side):
            with _ext.capture_safe_gc(), torch.cuda.graph(entry["graph"], stream=side):
                entry.update(build())
        torch.cuda.current_stream().wait_stream(side)
        self._graphs[key] = entry
        return entry

    def _graph_step_normal(self, idx: torch.Tensor, labels: torch.Tensor, scale: float) -> torch.Tensor:
        key = ("normal", tuple(idx.shape), scale)
        entry = self._graphs.get(key)
        if entry is None:
            static_idx, static_lab = idx.clone(), labels.clone()

            def build():
                loss = self._loss_normal(static_idx, static_lab)
                (loss * scale if scale != 1.0 else loss).backward()
                return {"idx": static_idx, "labels": static_lab, "loss": loss.detach()}

            entry = self._capture(key, build)
        entry["idx"].copy_(idx)
        entry["labels"].copy_(labels)
        entry["graph"].replay()
        return entry["loss"].clone()

    def _graph_chunk(self, ids_c, lab_c, shift, wkv, factor: float):
        """One infctx chunk (forward, loss, backward of ``loss * factor``) replayed from a graph; states in and out
        are static tensors.  Returns ``(loss, new_shift, new_wkv)`` (the state outputs are overwritten by the next
        replay, so the caller consumes them before calling again)."""
        m, cfg = self.model, self.cfg
        key = ("chunk", tuple(ids_c.shape), factor)
        entry = self._graphs.get(key)
        if entry is None:
            s_ids, s_lab, s_shift, s_wkv = ids_c.clone(), lab_c.clone(), shift.clone(), wkv.clone()

            def build():
                x, n_shift, n_wkv = m.forward_hidden_infctx(s_ids, s_shift, s_wkv, checkpoint=bool(cfg.grad_cp))
                Bc, Tc, C = x.shape
                loss_c = ops.linear_cross_entropy(x.reshape(Bc * Tc, C), m._head_weight(), s_lab.reshape(-1),
                                                  l2wrap=cfg.l2wrap, l2wrap_tokens=Bc * Tc)
                (loss_c * factor).backward()
                return {"ids": s_ids, "labels": s_lab, "shift": s_shift, "wkv": s_wkv, "loss": loss_c.detach(),
                        "new_shift": n_shift.detach(), "new_wkv": n_wkv.detach()}

            entry = self._capture(key, build)
        entry["ids"].copy_(ids_c)
        entry["labels"].copy_(lab_c)
        entry["shift"].copy_(shift)
        entry["wkv"].copy_(wkv)
        entry["graph"].replay()
        return entry["loss"], entry["new_shift"], entry["new_wkv"]

    # ------------------------------------------------------------------ one micro-batch
    def train_step(self, idx: torch.Tensor, labels: torch.Tensor, lr: float) -> torch.Tensor:
        """Forward + backward for one micro-batch; runs the optimiser every
        ``accumulate_grad_batches`` calls.  Returns the detached loss (device tensor)."""
        acc = self.cfg.accumulate_grad_batches
        scale = 1.0 / acc
        boundary = (self.micro_step + 1) % acc == 0
        with self.phases.phase("forward_backward"):
            if self.cfg.train_type == "infctx":
                loss = self._step_infctx(idx, labels, scale)
            elif self._graph_ok():
                loss = self._graph_step_normal(idx, labels, scale)
            else:
                loss = self._loss_normal(idx, labels)
                self.opt.arm()          # gradient buckets are reduced while backward is still running
                (loss * scale if acc > 1 else loss).backward()
                loss = loss.detach()
        with self.phases.phase("reduce_optimizer"):
            self.opt.finish_micro(boundary)
            if self.zero3 is not None:
                self.zero3.finish_micro()
            self.micro_step += 1
            self.tokens_seen += idx.numel()
            if boundary:
                self.opt.step(lr)
                self.opt.zero_grad()
                self.optimizer_steps += 1
                ops.bump_param_epoch()
        return loss

    def backward_and_step(self, loss: torch.Tensor, lr: float) -> bool:
        """Back-propagate an externally computed loss (already a mean over the micro-batch) and run the
        optimiser on accumulation boundaries.  Returns True when an optimiser step happened."""
        acc = self.cfg.accumulate_grad_batches
        boundary = (self.micro_step + 1) % acc == 0
        with self.phases.phase("backward"):
            (loss / acc if acc > 1 else loss).backward()
        with self.phases.phase("reduce_optimizer"):
            self.opt.finish_micro(boundary)
            if self.zero3 is not None:
                self.zero3.finish_micro()
            self.micro_step += 1
            if boundary:
                self.opt.step(lr)
                self.opt.zero_grad()
                self.optimizer_steps += 1
                ops.bump_param_epoch()
        return boundary

    def train_step_from_host(self, idx_cpu: torch.Tensor, labels_cpu: torch.Tensor, lr: float) -> float:
        """The call a trainer makes per batch: pinned host tensors in, Python float out.  Reading the loss waits for
        the step's kernels, so the device status words of the step are checked right after it at no extra cost."""
        idx = idx_cpu.to(self.ctx.device, non_blocking=True)
        labels = labels_cpu.to(self.ctx.device, non_blocking=True)
        if self.guard is not None:
            self.guard.before_step()
        loss = float(self.train_step(idx, labels, lr))
        if self.guard is not None:
            self.guard.after_step(self.health_ok())
        self.check_health()
        return loss

    # ------------------------------------------------------------------ health
    def start_guard(self, timeout_s: float = 60.0):
        """Multi-rank runs: start this rank's heartbeat and return the :class:`StepGuard` that ``train_step_from_host``
        consults around every step (peers alive before the step, all ranks' device status clean after it)."""
        if self.ctx.world_size <= 1 or self.guard is not None:
            return self.guard
        from .watchdog import StepGuard

        store = self.ctx.store()
        if store is None:
            return None
        self.guard = StepGuard(store, self.ctx.rank, self.ctx.world_size, agree=self.ctx.all_agree, timeout_s=timeout_s)
        self.guard.start()
        self.ctx.barrier()    # every rank has published its first heartbeat before anyone checks
        return self.guard

    def health_ok(self) -> bool:
        """False when a bounded wait inside one of the kernels expired during a finished step."""
        try:
            self.check_health()
        except RuntimeError:
            return False
        return True

    def check_health(self) -> None:
        """Raises when a device-side wait (peer flag, panel arrival, mbarrier) expired during a finished step.  Reads
        pinned host copies refreshed at the end of every step: no device synchronisation."""
        self.opt.check_health()
        if self.zero3 is not None:
            from ..ops import gemm_native

            self.zero3.check()
            code = gemm_native.check_status_nosync(self.ctx.device)
            if code:
                raise RuntimeError(f"rank {self.ctx.rank}: a wait inside the all-gather GEMM expired (code {code})")
