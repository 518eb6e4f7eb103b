"""ZeRO-3 for the large projection matrices: K-panel sharding with the all-gather fused into the GEMM.

What the reference gets from ``strategy="deepspeed_stage_3"`` (per-submodule parameter all-gather before
forward, backward and checkpoint recompute; ``rwkvtune/training/sft_trainer.py:457-458``) is done here
per weight matrix: ``att.receptance/key/value/output`` and ``ffn.key/value`` (99 % of a block's
parameters) are split into ``world`` column panels, rank ``p`` keeping ``W[:, p*K/W:(p+1)*K/W]`` in
symmetric memory.  The forward projection runs :func:`ag_mm_nt`, whose copy CTAs pull the panels over
NVLink into a local staging matrix while its MMA CTAs already multiply the panels that have landed.
The staged matrix is reused by the backward ``dy @ W`` of the same layer (with activation
checkpointing the recompute forward re-stages it immediately before that backward).

Scope: frozen weights (LoRA fine-tuning, the configuration the reference documents for stage 3).
Trainable full-rank weights under a stage-3 strategy stay replicated in bf16 with sharded optimiser
state (stage-2 behaviour): on 180 GB parts the bf16 copy of every supported model size fits.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import gemm, gemm_native

TARGETS = ("att.receptance", "att.key", "att.value", "att.output", "ffn.key", "ffn.value")


class ShardedWeight:
    """One ``[N, K]`` weight held as a K-panel per rank, plus access to a shared staging slot."""

    def __init__(self, owner: "Zero3ShardedLinears", name: str, slot: str, weight: torch.Tensor):
        import torch.distributed._symmetric_memory as symm_mem

        ctx = owner.ctx
        self.owner, self.name, self.slot = owner, name, slot
        self.N, self.K = weight.shape
        W, r = ctx.world_size, ctx.rank
        if self.K % W or (self.K // W) % 64:
            raise ValueError(f"{name}: K={self.K} cannot be split into {W} panels of a multiple of 64 columns")
        Kp = self.K // W
        self._flat = symm_mem.empty(self.N * Kp, dtype=torch.bfloat16, device=ctx.device)
        self.panel = self._flat.view(self.N, Kp)
        self.panel.copy_(weight[:, r * Kp:(r + 1) * Kp].to(torch.bfloat16))
        self.handle = symm_mem.rendezvous(self._flat, dist.group.WORLD.group_name)
        self.ptrs = list(self.handle.buffer_ptrs)

    def gathered(self) -> gemm_native.GatheredWeight:
        return self.owner.staging_slot(self)

    def full_weight(self) -> torch.Tensor:
        """The staged full matrix, re-gathered (plain peer copies) if another layer used the slot since."""
        gw = self.gathered()
        if gw.current_owner is not self:
            Kp = self.K // self.owner.ctx.world_size
            for p in range(self.owner.ctx.world_size):
                src = self.handle.get_buffer(p, (self.N, Kp), torch.bfloat16)
                gw.staged[:, p * Kp:(p + 1) * Kp].copy_(src)
            gw.current_owner = self
        return gw.staged


class _AGLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sw: ShardedWeight):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        gw = sw.gathered()
        gw.ptrs_for(sw)
        y = gemm_native.ag_mm_nt(x2, gw)
        gw.current_owner = sw
        ctx.sw, ctx.shape = sw, x.shape
        return y.reshape(*x.shape[:-1], sw.N)

    @staticmethod
    def backward(ctx, dy):
        sw = ctx.sw
        dy2 = dy.reshape(-1, dy.shape[-1])
        return gemm.mm_nn(dy2 if dy2.is_contiguous() else dy2.contiguous(), sw.full_weight()).reshape(ctx.shape), None


class _LoraAGLinearFn(torch.autograd.Function):
    """``x W^T + s (x A^T) B^T`` with ``W`` sharded and frozen."""

    @staticmethod
    def forward(ctx, x, sw: ShardedWeight, a, b, scaling: float):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        gw = sw.gathered()
        gw.ptrs_for(sw)
        base = gemm_native.ag_mm_nt(x2, gw)
        gw.current_owner = sw
        xa = gemm.mm_nt(x2, a)
        y = gemm.addmm_nt_(base, xa * scaling, b)
        ctx.save_for_backward(x2, a, b, xa)
        ctx.sw, ctx.shape, ctx.scaling = sw, x.shape, scaling
        return y.reshape(*x.shape[:-1], sw.N)

    @staticmethod
    def backward(ctx, dy):
        x2, a, b, xa = ctx.saved_tensors
        s, sw = ctx.scaling, ctx.sw
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dyb = gemm.mm_nn(dy2, b)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm.addmm_nn_(gemm.mm_nn(dy2, sw.full_weight()), dyb * s, a).reshape(ctx.shape)
        da = gemm.mm_tn(dyb, x2) * s if ctx.needs_input_grad[2] else None
        db = gemm.mm_tn(dy2, xa) * s if ctx.needs_input_grad[3] else None
        return dx, None, da, db, None


class _Slot(gemm_native.GatheredWeight):
    def __init__(self, rank, world, N, K, device, n_copy):
        super().__init__([0] * world, rank, world, N, K, device, n_copy)
        self.current_owner = None

    def ptrs_for(self, sw: ShardedWeight) -> None:
        for i, p in enumerate(sw.ptrs):
            self.ptrs[i] = int(p)


class Zero3ShardedLinears:
    def __init__(self, model: nn.Module, ctx, n_copy: int = 16):
        from ..peft.lora.layer import LoraLinear

        self.ctx = ctx
        self.n_copy = n_copy
        self._slots: Dict[str, _Slot] = {}
        self.sharded: List[ShardedWeight] = []
        freed = 0
        for name, module in model.named_modules():
            role = next((t for t in TARGETS if name.endswith(t)), None)
            if role is None:
                continue
            lin = module.base_layer if isinstance(module, LoraLinear) else module
            if not isinstance(lin, nn.Linear) or lin.weight.requires_grad:
                continue
            sw = ShardedWeight(self, name, role, lin.weight.data)
            self.sharded.append(sw)
            freed += lin.weight.numel()
            lin.weight.data = torch.empty(0, dtype=lin.weight.dtype, device=lin.weight.device)
            module._sharded = sw
        self.freed_elements = freed
        torch.cuda.synchronize()
        if ctx.world_size > 1:
            dist.barrier()

    def staging_slot(self, sw: ShardedWeight) -> _Slot:
        key = f"{sw.slot}:{sw.N}x{sw.K}"
        if key not in self._slots:
            self._slots[key] = _Slot(self.ctx.rank, self.ctx.world_size, sw.N, sw.K, self.ctx.device, self.n_copy)
        return self._slots[key]

    def materialize(self, model: nn.Module) -> None:
        """Put full weights back into the modules (used before saving merged/full checkpoints)."""
        for name, module in model.named_modules():
            sw = getattr(module, "_sharded", None)
            if sw is None:
                continue
            lin = module.base_layer if hasattr(module, "base_layer") else module
            lin.weight.data = sw.full_weight().clone()
            module._sharded = None


def ag_linear(x: torch.Tensor, sw: ShardedWeight) -> torch.Tensor:
    return _AGLinearFn.apply(x, sw)


def lora_ag_linear(x: torch.Tensor, sw: ShardedWeight, a: torch.Tensor, b: torch.Tensor, scaling: float) -> torch.Tensor:
    return _LoraAGLinearFn.apply(x, sw, a, b, scaling)
