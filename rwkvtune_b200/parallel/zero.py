"""Sharded optimiser over a :class:`FlatParamSpace` (ZeRO stages 0/1/2; stage 3 builds on it).

What the reference delegates to Lightning + DeepSpeed by a strategy string
(``rwkvtune/training/sft_config.py:112``; ``strategy="deepspeed_stage_2"`` etc.) is owned here:

* stage 0 ("ddp"/"auto"): gradients all-reduced, optimiser state replicated;
* stage 1/2 ("deepspeed_stage_2"): gradients reduce-scattered, fp32 master weights and Adam
  moments exist only for the owned shard, updated bf16 parameters all-gathered.

Two transports implement the same interface: ``"nccl"`` issues torch.distributed collectives
(the baseline) and ``"p2p"`` runs the fused reduce-scatter + AdamW + broadcast kernels over
peer-mapped memory (:mod:`rwkvtune_b200.parallel.p2p`).  On CPU (gloo ranks) the arithmetic
uses the PyTorch statements of the same kernels, which is how the partitioning logic is
tested without GPUs.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import reference as ref
from .bootstrap import DistContext
from .flat import FlatParamSpace


class ZeroOptimizer:
    def __init__(self, space: FlatParamSpace, ctx: DistContext, stage: int = 0, betas=(0.9, 0.99),
                 eps: float = 1e-8, grad_clip: float = 1.0, transport: str = "nccl"):
        self.space, self.ctx = space, ctx
        self.stage = stage if ctx.world_size > 1 else 0
        self.beta1, self.beta2 = betas
        self.eps, self.grad_clip = eps, grad_clip
        self.transport = transport
        self.step_count = 0
        if self.stage >= 1:
            self.lo, self.hi = space.shard_range(ctx.rank)
        else:
            self.lo, self.hi = 0, space.padded
        dev = space.device
        self.master = space.params[self.lo:self.hi].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._scratch = torch.zeros(1024, dtype=torch.float32, device=dev)
        self._shard_grad = (torch.empty(self.hi - self.lo, dtype=space.dtype, device=dev)
                            if self.stage >= 1 else None)
        self._p2p = None
        if transport == "p2p" and ctx.world_size > 1 and self.stage >= 1 and space.device.type == "cuda":
            from . import p2p

            self._p2p = p2p.FusedZero2(space, ctx, self)
        self.last_grad_norm: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ pieces
    def _local_grad(self) -> torch.Tensor:
        return self._shard_grad if self.stage >= 1 else self.space.grads

    def _reduce_gradients(self) -> float:
        """Returns the factor the (summed) gradient still has to be multiplied by."""
        W = self.ctx.world_size
        if W == 1:
            return 1.0
        g = self.space.grads
        if self.stage == 0:
            dist.all_reduce(g)
        elif self.ctx.backend == "nccl":
            dist.reduce_scatter_tensor(self._shard_grad, g)
        else:   # gloo has no reduce_scatter: all-reduce and slice
            dist.all_reduce(g)
            self._shard_grad.copy_(g[self.lo:self.hi])
        return 1.0 / W

    def _grad_norm_sq(self, scale: float) -> None:
        g = self._local_grad()
        if g.is_cuda:
            from ..ops import _ext

            _ext.call("rwkv_grad_sumsq_bf16" if g.dtype == torch.bfloat16 else "rwkv_grad_sumsq_bf16",
                      _ext.ptr(g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)), _ext.i64(g.numel()),
                      _ext.f32(scale), _ext.ptr(self._scratch), _ext.ptr(self.norm_sq), _ext.i32(0), _ext.stream())
        else:
            from ..ops import cpu_ops

            self.norm_sq.copy_(cpu_ops.grad_norm_sq(g, scale).reshape(1))
        if self.stage >= 1:
            dist.all_reduce(self.norm_sq)

    def _adam(self, lr: float, scale: float) -> None:
        sp = self.space
        g = self._local_grad()
        self.step_count += 1
        for gi, s, e in sp.group_segments_in(self.lo, self.hi):
            grp = sp.groups[gi]
            a, b = s - self.lo, e - self.lo
            p_out = sp.params[s:e]
            if g.is_cuda and sp.dtype == torch.bfloat16:
                from ..ops import _ext

                _ext.call("rwkv_adamw_step", _ext.ptr(self.master[a:b]), _ext.ptr(self.exp_avg[a:b]),
                          _ext.ptr(self.exp_avg_sq[a:b]), _ext.ptr(g[a:b]), _ext.i32(0), _ext.ptr(p_out),
                          _ext.i64(b - a), _ext.ptr(self.norm_sq if self.grad_clip > 0 else None),
                          _ext.f32(lr * grp.lr_scale), _ext.f32(self.beta1), _ext.f32(self.beta2), _ext.f32(self.eps),
                          _ext.f32(grp.weight_decay), _ext.i32(self.step_count), _ext.f32(scale),
                          _ext.f32(self.grad_clip), _ext.stream())
            else:
                coef = scale
                if self.grad_clip > 0:
                    nrm = float(self.norm_sq.sqrt())
                    coef *= min(1.0, self.grad_clip / (nrm + 1e-6))
                if g.is_cuda:
                    ref.adamw_step(self.master[a:b], g[a:b], self.exp_avg[a:b], self.exp_avg_sq[a:b], lr * grp.lr_scale,
                                   self.beta1, self.beta2, self.eps, grp.weight_decay, self.step_count, coef)
                else:
                    from ..ops import cpu_ops

                    if getattr(self, "_cpu_scratch", None) is None or self._cpu_scratch.numel() < b - a:
                        self._cpu_scratch = torch.empty(self.hi - self.lo, dtype=torch.float32)
                    cpu_ops.adamw_step(self.master[a:b], g[a:b], self.exp_avg[a:b], self.exp_avg_sq[a:b],
                                       lr * grp.lr_scale, self.beta1, self.beta2, self.eps, grp.weight_decay,
                                       self.step_count, coef, self._cpu_scratch[:b - a])
                p_out.copy_(self.master[a:b])

    def _gather_params(self) -> None:
        if self.stage < 1:
            return
        sp = self.space
        if self.ctx.backend == "nccl":
            dist.all_gather_into_tensor(sp.params, sp.params[self.lo:self.hi])
        else:
            parts = [torch.empty(sp.shard_numel, dtype=sp.dtype, device=sp.device) for _ in range(self.ctx.world_size)]
            dist.all_gather(parts, sp.params[self.lo:self.hi].clone())
            sp.params.copy_(torch.cat(parts))

    # ------------------------------------------------------------------ public
    def arm(self) -> None:
        """Before the backward pass of a micro-batch whose every parameter receives exactly one gradient: lets the
        fused transport reduce gradient buckets while backward is still running.  No effect on other transports."""
        if self._p2p is not None:
            self._p2p.arm()

    def finish_micro(self, boundary: bool) -> None:
        """After the backward pass of a micro-batch.  Fused transport: whatever was not reduced during backward goes
        out now, micro-batches are summed in fp32 on the owning rank, and on a non-boundary micro-batch the local
        bf16 gradient buffer is cleared.  Library transports keep accumulating micro-batches in the flat bf16
        gradient buffer and reduce once at the boundary (the gradient of one micro-batch is already a sum over
        thousands of tokens; adding up to 16 of them in bf16 costs at most half an ulp each)."""
        if self._p2p is not None:
            self._p2p.finish_micro(boundary)

    def check_health(self) -> None:
        """Raise if a bounded device-side wait expired during a finished step (no device synchronisation)."""
        if self._p2p is not None:
            self._p2p.check()

    def step(self, lr: float, grad_scale: float = 1.0) -> None:
        """Reduce gradients, clip by global norm, AdamW on the owned range, publish new parameters.

        ``grad_scale`` multiplies the summed gradient (``1 / accumulate_grad_batches`` when the loss
        was not pre-divided)."""
        if self._p2p is not None:
            self._p2p.step(lr, grad_scale)
            return
        scale = self._reduce_gradients() * grad_scale
        if self.grad_clip > 0:
            self._grad_norm_sq(scale)
            self.last_grad_norm = self.norm_sq
        self._adam(lr, scale)
        self._gather_params()

    def zero_grad(self) -> None:
        self.space.zero_grads()

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> Dict[str, object]:
        return {"step": self.step_count, "lo": self.lo, "hi": self.hi, "world_size": self.ctx.world_size,
                "stage": self.stage, "padded": self.space.padded, "numel": self.space.numel,
                "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu()}

    def load_full_state(self, master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, step: int) -> None:
        """Load from *unsharded* fp32 vectors of length ``space.numel`` (re-sharding is a slice)."""
        n = self.space.numel
        for dst, src in ((self.master, master), (self.exp_avg, exp_avg), (self.exp_avg_sq, exp_avg_sq)):
            dst.zero_()
            s, e = self.lo, min(self.hi, n)
            if s < e:
                dst[: e - s].copy_(src[s:e])
        self.step_count = int(step)
        self.space.params[self.lo:self.hi].copy_(self.master)
        self._gather_params()


def merge_shards(shards: List[Dict[str, object]]):
    """Concatenate per-rank optimiser shards (in rank order) into unsharded fp32 vectors."""
    shards = sorted(shards, key=lambda s: s["lo"])
    numel = shards[0]["numel"]
    cat = lambda k: torch.cat([s[k] for s in shards])[:numel]
    return cat("master"), cat("exp_avg"), cat("exp_avg_sq"), shards[0]["step"]
