"""ZeRO-3 for the large projection matrices: K-panel sharding, the all-gather fused into the GEMM, the weight
gradient reduce-scattered to the panel owners during backward, optimiser state per panel.

What the reference gets from ``strategy="deepspeed_stage_3"`` (every parameter partitioned, gathered per submodule
before forward, backward and checkpoint recompute, gradients reduce-scattered, a consolidated ``model.pth`` on save;
``rwkvtune/training/sft_trainer.py:455-458``, ``rwkvtune/training/callbacks.py:385-426``) is done here per weight
matrix: ``att.receptance/key/value/output`` and ``ffn.key/value`` (99 % of a block's parameters) are split into
``world`` column panels, rank ``p`` keeping ``W[:, p*K/W:(p+1)*K/W]``.  All panels of a rank live in one
symmetric-memory buffer, so every rank holds device pointers to every peer's panels.

* **Forward**: :func:`gemm_native.ag_mm_nt` - four copy warps in every CTA of the GEMM pull the panels over NVLink
  into a local staging matrix, 256 weight rows at a time, while the tensor-core warps already multiply the column
  tiles whose weight rows have landed.
* **Backward, data gradient**: ``dy @ W`` needs the full matrix again.  With activation checkpointing the recompute
  forward has just staged it.  Otherwise the staging slot of that role holds the next layer's matrix, and this
  layer's is brought in by :func:`prefetch`: a gather kernel of this repository on a side stream, issued as soon as
  the next layer's backward has consumed the slot, so the transfer runs under that layer's remaining backward work.
* **Backward, weight gradient** (trainable matrices): every rank forms its full ``dW = dy^T x`` into a symmetric
  staging buffer and raises a flag; each owner then sums its column panel of all ranks' ``dW`` (fixed rank order,
  fp32, accumulated over micro-batches) on the side stream and raises a "consumed" flag that frees the staging
  buffer for the layer after next.
* **Optimiser**: fp32 master weights and Adam moments exist only for the owned panels; the update writes the new
  bf16 panel in place, where the peers' next gather finds it (no parameter broadcast).  The global gradient norm
  includes the panels: their squared norm is added to this rank's share before the ranks exchange shares.

Frozen matrices (LoRA fine-tuning) use the forward and data-gradient parts only.  Embedding, head and the small
per-channel parameters stay in the flat ZeRO-2 space (replicated bf16 copy, sharded optimiser state).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _ext, gemm, gemm_native

TARGETS = ("att.receptance", "att.key", "att.value", "att.output", "ffn.key", "ffn.value")
FLAG_WORD0 = 128          # flag words of weight i: ready = FLAG_WORD0 + 32 i, consumed = FLAG_WORD0 + 32 i + 16
REDUCE_BLOCKS = 512


def _arr(ptrs):
    return (ctypes.c_ulonglong * len(ptrs))(*[int(p) for p in ptrs])


class ShardedWeight:
    """One ``[N, K]`` weight held as a K-panel per rank."""

    def __init__(self, owner: "Zero3ShardedLinears", index: int, name: str, slot: str, N: int, K: int, trainable: bool):
        self.owner, self.index, self.name, self.slot = owner, index, name, slot
        self.N, self.K, self.trainable = N, K, trainable
        self.Kp = K // owner.ctx.world_size
        self.panel: Optional[torch.Tensor] = None        # [N, Kp] bf16 view into the rank's symmetric panel buffer
        self.ptrs = None                                  # ctypes array: every rank's panel address in this process
        self.gacc: Optional[torch.Tensor] = None          # [N, Kp] fp32 gradient accumulator (trainable only)
        self.order_in_slot = 0
        import re

        m = re.search(r"blocks\.(\d+)\.", name)
        self.layer = int(m.group(1)) if m else 0
        self.anchor = torch.empty(0, device=owner.ctx.device, requires_grad=True) if trainable else None

    def gathered(self) -> "_Slot":
        return self.owner.staging_slot(self)

    def full_weight(self) -> torch.Tensor:
        """The staged full matrix; gathered now (gather kernel, current stream) unless the slot already holds it or
        a prefetch of it is in flight."""
        gw = self.gathered()
        if gw.current_owner is self:
            if gw.pending is not None:     # a prefetch on the side stream: make the current stream wait for it
                torch.cuda.current_stream().wait_event(gw.pending)
                gw.pending = None
            return gw.staged
        self.owner.gather_into(self, gw, _ext.stream())
        gw.current_owner = self
        gw.pending = None
        return gw.staged


class _AGLinearFn(torch.autograd.Function):
    """``x W^T`` with ``W`` sharded.  ``anchor`` is an empty tensor that requires grad when ``W`` is trainable, so that
    the node is part of the graph even if ``x`` needs no gradient; the weight gradient is not returned to autograd
    but reduce-scattered to the panel owners from inside ``backward``."""

    @staticmethod
    def forward(ctx, x, sw: ShardedWeight, anchor):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        y = sw.owner.forward_gemm(x2, sw)
        ctx.sw, ctx.shape = sw, x.shape
        if sw.trainable:
            ctx.save_for_backward(x2)
        return y.reshape(*x.shape[:-1], sw.N)

    @staticmethod
    def backward(ctx, dy):
        sw = ctx.sw
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm.mm_nn(dy2, sw.full_weight()).reshape(ctx.shape)
        sw.owner.after_dgrad(sw)
        if sw.trainable:
            (x2,) = ctx.saved_tensors
            sw.owner.weight_gradient(sw, dy2, x2)
        return dx, None, None


class _LoraAGLinearFn(torch.autograd.Function):
    """``x W^T + s (x A^T) B^T`` with ``W`` sharded and frozen."""

    @staticmethod
    def forward(ctx, x, sw: ShardedWeight, a, b, scaling: float, residual=None, act=None):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        xa_s = (gemm.mm_nt(x2, a) * scaling).contiguous()        # scaled once: used here and by dB
        b_c = b if b.is_contiguous() else b.contiguous()
        r2 = None if residual is None else residual.reshape(-1, residual.shape[-1])
        if xa_s.shape[1] % 8 == 0 and b_c.dtype == torch.bfloat16 and (r2 is None or (
                r2.dtype == torch.bfloat16 and r2.stride(1) == 1 and r2.data_ptr() % 16 == 0 and r2.stride(0) % 8 == 0)):
            # the adapter term is the last K block of the all-gather GEMM (no second pass over y); relu^2 or the
            # residual sum in the same launch's epilogue
            y = sw.owner.forward_gemm(x2, sw, extra=(xa_s, b_c), epilogue=1 if act else 0, residual=r2)
        else:
            y = gemm.addmm_nt_(sw.owner.forward_gemm(x2, sw), xa_s, b)
            if act:
                y = torch.relu(y) ** 2
            if r2 is not None:
                y = y + r2
        ctx.save_for_backward(x2, a, b, xa_s, y if act else None)
        ctx.sw, ctx.shape, ctx.scaling, ctx.act = sw, x.shape, scaling, act
        return y.reshape(*x.shape[:-1], sw.N)

    @staticmethod
    def backward(ctx, dy):
        from ..peft.lora.layer import _relu_sq_grad

        x2, a, b, xa_s, y = ctx.saved_tensors
        s, sw = ctx.scaling, ctx.sw
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dpre = _relu_sq_grad(y, dy2) if ctx.act else dy2
        dyb_s = gemm.mm_nn(dpre, b) * s                          # scaled once: used by dx and by dA
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm.mm_nn_plus(dpre, sw.full_weight(), dyb_s, a).reshape(ctx.shape)
        sw.owner.after_dgrad(sw)
        da = gemm.mm_tn(dyb_s, x2) if ctx.needs_input_grad[2] else None
        db = gemm.mm_tn(dpre, xa_s) if ctx.needs_input_grad[3] else None
        d_res = dy if (len(ctx.needs_input_grad) > 5 and ctx.needs_input_grad[5]) else None
        return dx, None, da, db, None, d_res, None


class _Slot(gemm_native.GatheredWeight):
    """Staging matrix shared by all weights of one role and shape (one is live at a time)."""

    def __init__(self, rank, world, N, K, device, n_copy):
        super().__init__([0] * world, rank, world, N, K, device, n_copy)
        self.current_owner: Optional[ShardedWeight] = None
        self.pending: Optional[torch.cuda.Event] = None     # completion of a prefetch into this slot
        self.members: List[ShardedWeight] = []               # weights using this slot, in forward order
        self.dw_stage: List[torch.Tensor] = []               # two symmetric [N, K] bf16 buffers for weight gradients
        self.dw_ptrs: List[object] = []
        self.dw_last_user: List[Optional[ShardedWeight]] = [None, None]
        self.dw_next = 0

    def ptrs_for(self, sw: ShardedWeight) -> None:
        for i in range(self.world):
            self.ptrs[i] = sw.ptrs[i]


class Zero3ShardedLinears:
    def __init__(self, model: nn.Module, ctx, n_copy: int = 16, shard_trainable: bool = True, timeout_s: float = 20.0):
        import torch.distributed._symmetric_memory as symm_mem

        from ..peft.lora.layer import LoraLinear

        self.ctx, self.n_copy = ctx, n_copy
        W, r, dev = ctx.world_size, ctx.rank, ctx.device
        self._slots: Dict[str, _Slot] = {}
        self.sharded: List[ShardedWeight] = []
        found = []
        for name, module in model.named_modules():
            role = next((t for t in TARGETS if name.endswith(t)), None)
            if role is None:
                continue
            lin = module.base_layer if isinstance(module, LoraLinear) else module
            if not isinstance(lin, nn.Linear) or lin.weight.numel() == 0:
                continue
            trainable = bool(lin.weight.requires_grad)
            if trainable and (not shard_trainable or isinstance(module, LoraLinear)):
                continue
            N, K = lin.weight.shape
            if K % W or (K // W) % 64:
                raise ValueError(f"{name}: K={K} cannot be split into {W} panels of a multiple of 64 columns")
            found.append((name, role, module, lin, trainable, N, K))
        total = sum(N * (K // W) for *_, N, K in found)
        group = dist.group.WORLD.group_name
        self.panels = symm_mem.empty(max(total, 8), dtype=torch.bfloat16, device=dev)
        n_flags = FLAG_WORD0 + 32 * max(len(found), 1)
        self.ctrl = symm_mem.empty(n_flags, dtype=torch.int32, device=dev)
        self.ctrl.zero_()
        off, offsets = 0, []
        freed = 0
        for i, (name, role, module, lin, trainable, N, K) in enumerate(found):
            sw = ShardedWeight(self, i, name, role, N, K, trainable)
            Kp = K // W
            sw.panel = self.panels[off:off + N * Kp].view(N, Kp)
            sw.panel.copy_(lin.weight.data[:, r * Kp:(r + 1) * Kp].to(torch.bfloat16))
            offsets.append(off)
            off += N * Kp
            freed += lin.weight.numel()
            lin.weight.data = torch.empty(0, dtype=lin.weight.dtype, device=lin.weight.device)
            lin.weight.requires_grad_(False)      # the panel is what is trained; nothing flows to the empty tensor
            module._sharded = sw
            self.sharded.append(sw)
        torch.cuda.synchronize()
        dist.barrier()
        self._h_panels = symm_mem.rendezvous(self.panels, group)
        self._h_ctrl = symm_mem.rendezvous(self.ctrl, group)
        base = [int(p) for p in self._h_panels.buffer_ptrs]
        self.ctrl_ptrs = _arr(list(self._h_ctrl.buffer_ptrs))
        for sw, o in zip(self.sharded, offsets):
            sw.ptrs = _arr([b + 2 * o for b in base])
        self.freed_elements = freed
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.timeout_ns = int(timeout_s * 1e9)
        self.side = torch.cuda.Stream(device=dev)            # weight-gradient exchange (bounded flag waits + sums)
        self.side_gather = torch.cuda.Stream(device=dev)     # prefetch gathers for the data-gradient GEMMs
        self.prefetch = True
        self.recompute_below = 0      # layers with a smaller index are recomputed in backward (their forward re-stages)
        self.flag_epoch = 0           # one epoch per backward pass of a micro-batch
        self._epoch_open = False
        # ---- slots (staging matrices) and, for trainable weights, optimiser state per panel
        for sw in self.sharded:
            slot = self.staging_slot(sw)
            sw.order_in_slot = len(slot.members)
            slot.members.append(sw)
        self.trainable = [sw for sw in self.sharded if sw.trainable]
        self.opt_state = None
        if self.trainable:
            n_train = sum(sw.N * sw.Kp for sw in self.trainable)
            self.gacc = torch.zeros(n_train, dtype=torch.float32, device=dev)
            self.master = torch.empty(n_train, dtype=torch.float32, device=dev)
            self.exp_avg = torch.zeros(n_train, dtype=torch.float32, device=dev)
            self.exp_avg_sq = torch.zeros(n_train, dtype=torch.float32, device=dev)
            self.partials = torch.zeros(len(self.trainable) * REDUCE_BLOCKS, dtype=torch.float32, device=dev)
            self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            self.norm_total = torch.zeros(1, dtype=torch.float32, device=dev)
            o = 0
            for j, sw in enumerate(self.trainable):
                n = sw.N * sw.Kp
                sw.gacc = self.gacc[o:o + n]
                sw.train_off, sw.train_index = o, j
                self.master[o:o + n].copy_(sw.panel.reshape(-1).float())
                o += n
            for slot in self._slots.values():
                if any(m.trainable for m in slot.members):
                    for _ in range(2):
                        buf = symm_mem.empty(slot.N * slot.K, dtype=torch.bfloat16, device=dev)
                        buf.zero_()
                        slot.dw_stage.append(buf)
            torch.cuda.synchronize()
            dist.barrier()
            for slot in self._slots.values():
                slot.dw_ptrs = [_arr(list(symm_mem.rendezvous(buf, group).buffer_ptrs)) for buf in slot.dw_stage]
            self._accumulated = False
        torch.cuda.synchronize()
        dist.barrier()

    # ------------------------------------------------------------------ staging / gather
    def staging_slot(self, sw: ShardedWeight) -> _Slot:
        key = f"{sw.slot}:{sw.N}x{sw.K}"
        if key not in self._slots:
            self._slots[key] = _Slot(self.ctx.rank, self.ctx.world_size, sw.N, sw.K, self.ctx.device, self.n_copy)
        return self._slots[key]

    def forward_gemm(self, x2: torch.Tensor, sw: ShardedWeight, extra=None, epilogue: int = 0, residual=None) -> torch.Tensor:
        """``x2 @ W^T`` with the gather fused in; ``extra = (u [M, r], v [N, r])`` adds ``u @ v^T`` inside the same launch;
        ``epilogue=1`` applies relu(.)^2, ``residual [M, N]`` is added, both in that launch's epilogue."""
        gw = sw.gathered()
        if gw.pending is not None:      # a prefetch may still be writing the slot
            torch.cuda.current_stream().wait_event(gw.pending)
            gw.pending = None
        gw.ptrs_for(sw)
        if extra is None and not epilogue and residual is None:
            y = gemm_native.ag_mm_nt(x2, gw)
        else:
            u, v = extra if extra is not None else (None, None)
            y = gemm_native.ag_mm_nt(x2, gw, u, v, epilogue=epilogue, residual=residual)
        gw.current_owner = sw
        return y

    def gather_into(self, sw: ShardedWeight, gw: _Slot, stream_handle, blocks: int = 64) -> None:
        _ext.call("rwkv_ag_gather", sw.ptrs, _ext.i32(self.ctx.rank), _ext.i32(self.ctx.world_size), _ext.i32(sw.N),
                  _ext.i32(sw.K), _ext.ptr(gw.staged), _ext.i32(blocks), stream_handle)

    def after_dgrad(self, sw: ShardedWeight) -> None:
        """The data-gradient GEMM of ``sw`` has been queued: its slot is free for the matrix that the backward pass
        needs next in this slot - the same role one layer down.  Gather it on the side stream now."""
        gw = sw.gathered()
        if not self.prefetch or sw.order_in_slot == 0 or gw.current_owner is not sw:
            return
        prev = gw.members[sw.order_in_slot - 1]
        if prev.layer < self.recompute_below:     # its recompute forward will stage it again anyway
            return
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream())
        self.side_gather.wait_event(done)
        self.gather_into(prev, gw, ctypes.c_void_p(self.side_gather.cuda_stream))
        landed = torch.cuda.Event()
        landed.record(self.side_gather)
        gw.current_owner, gw.pending = prev, landed

    # ------------------------------------------------------------------ weight gradient of a trainable panel
    def _ready_word(self, sw: ShardedWeight) -> int:
        return FLAG_WORD0 + 32 * sw.index

    def weight_gradient(self, sw: ShardedWeight, dy2: torch.Tensor, x2: torch.Tensor) -> None:
        if not self._epoch_open:
            self.flag_epoch += 1
            self._epoch_open = True
        slot = sw.gathered()
        which = slot.dw_next
        slot.dw_next ^= 1
        st = _ext.stream()
        W, rank = self.ctx.world_size, self.ctx.rank
        last = slot.dw_last_user[which]
        if last is not None:   # every rank must have finished summing the previous tenant of this buffer
            user, epoch = last
            _ext.call("rwkv_p2p_wait", self.ctrl_ptrs, _ext.i32(rank), _ext.i32(W), _ext.i32(self._ready_word(user) + 16),
                      _ext.i32(epoch), _ext.ptr(self.status), _ext.i64(self.timeout_ns), st)
        dw = slot.dw_stage[which].view(sw.N, sw.K)
        gemm.mm_tn_into(dw, dy2, x2)
        _ext.call("rwkv_p2p_signal", self.ctrl_ptrs, _ext.i32(rank), _ext.i32(W), _ext.i32(self._ready_word(sw)),
                  _ext.i32(self.flag_epoch), st)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.side.wait_event(ev)
        sst = ctypes.c_void_p(self.side.cuda_stream)
        _ext.call("rwkv_p2p_wait", self.ctrl_ptrs, _ext.i32(rank), _ext.i32(W), _ext.i32(self._ready_word(sw)),
                  _ext.i32(self.flag_epoch), _ext.ptr(self.status), _ext.i64(self.timeout_ns), sst)
        part = self.partials[sw.train_index * REDUCE_BLOCKS:(sw.train_index + 1) * REDUCE_BLOCKS]
        blocks = max(1, min(REDUCE_BLOCKS, (sw.N * sw.Kp // 8 + 255) // 256))
        _ext.call("rwkv_zero3_reduce_panel", slot.dw_ptrs[which], _ext.i32(rank), _ext.i32(W), _ext.i32(sw.N),
                  _ext.i32(sw.K), _ext.f32(1.0 / W), _ext.ptr(sw.gacc), _ext.ptr(part), _ext.i32(blocks),
                  _ext.i32(1 if self._accumulated else 0), _ext.ptr(self.status), sst)
        _ext.call("rwkv_p2p_signal", self.ctrl_ptrs, _ext.i32(rank), _ext.i32(W), _ext.i32(self._ready_word(sw) + 16),
                  _ext.i32(self.flag_epoch), sst)
        slot.dw_last_user[which] = (sw, self.flag_epoch)

    def finish_micro(self) -> None:
        """After the backward pass of a micro-batch: later micro-batches add to the panel gradients."""
        if self.trainable and self._epoch_open:
            self._epoch_open = False
            self._accumulated = True

    # ------------------------------------------------------------------ optimiser over the owned panels
    def attach(self, fused_zero2, weight_decay: float, betas, eps: float, grad_clip: float) -> None:
        """Couple the panel optimiser to the fused ZeRO-2 step of the remaining parameters: the panels' squared
        gradient norm joins this rank's norm share, and the panel update runs once the global norm is known."""
        self.weight_decay, self.betas, self.eps, self.grad_clip = weight_decay, betas, eps, grad_clip
        self.step_count = 0
        self._fz = fused_zero2
        fused_zero2.extra_sumsq = self.sumsq
        fused_zero2.before_publish = self._before_publish
        fused_zero2.after_norm = self._after_norm

    def _before_publish(self) -> None:
        joined = torch.cuda.Event()
        joined.record(self.side)
        torch.cuda.current_stream().wait_event(joined)
        torch.sum(self.partials, dim=0, keepdim=True, out=self.sumsq)

    def _after_norm(self, lr: float) -> None:
        W = self.ctx.world_size
        norms = self._fz.ctrl.view(torch.float32)[64:64 + W]
        torch.sum(norms, dim=0, keepdim=True, out=self.norm_total)
        self.step_count += 1
        # one launch over all owned panels: their bf16 values are contiguous in the symmetric panel buffer only per
        # weight, so the update walks weight by weight
        for sw in self.trainable:
            o, cnt = sw.train_off, sw.N * sw.Kp
            _ext.call("rwkv_adamw_step", _ext.ptr(self.master[o:o + cnt]), _ext.ptr(self.exp_avg[o:o + cnt]),
                      _ext.ptr(self.exp_avg_sq[o:o + cnt]), _ext.ptr(self.gacc[o:o + cnt]), _ext.i32(1),
                      _ext.ptr(sw.panel), _ext.i64(cnt), _ext.ptr(self.norm_total if self.grad_clip > 0 else None),
                      _ext.f32(lr), _ext.f32(self.betas[0]), _ext.f32(self.betas[1]), _ext.f32(self.eps),
                      _ext.f32(self.weight_decay), _ext.i32(self.step_count), _ext.f32(1.0), _ext.f32(self.grad_clip),
                      _ext.stream())
        self._accumulated = False
        for slot in self._slots.values():      # staged copies are stale now
            slot.current_owner = None
        self.status_host.copy_(self.status, non_blocking=True)
        gemm_native.snapshot_status(self.ctx.device)

    def check(self) -> None:
        code = int(self.status_host[0])
        if code:
            raise RuntimeError(f"rank {self.ctx.rank}: a wait for rank {code % 100} expired in the ZeRO-3 gradient exchange")

    # ------------------------------------------------------------------ state for checkpoints
    def state_dict(self) -> Dict[str, object]:
        out = {"world_size": self.ctx.world_size, "rank": self.ctx.rank, "step": getattr(self, "step_count", 0), "panels": {}}
        for sw in self.trainable:
            o, cnt = sw.train_off, sw.N * sw.Kp
            out["panels"][sw.name] = {k: t[o:o + cnt].view(sw.N, sw.Kp).cpu()
                                      for k, t in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq))}
        return out

    def load_state(self, shards: List[Dict[str, object]]) -> None:
        """``shards``: the ``state_dict`` of every rank of the run that saved (any world size).  Panels are
        re-assembled along the column dimension and re-cut for this world size."""
        shards = sorted(shards, key=lambda s: s["rank"])
        if len(shards) != shards[0]["world_size"]:
            raise RuntimeError(f"panel optimiser state of {shards[0]['world_size']} ranks, {len(shards)} files found")
        r, W = self.ctx.rank, self.ctx.world_size
        for sw in self.trainable:
            o, cnt = sw.train_off, sw.N * sw.Kp
            for key, dst in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                full = torch.cat([s["panels"][sw.name][key] for s in shards], dim=1)
                dst[o:o + cnt].copy_(full[:, r * sw.Kp:(r + 1) * sw.Kp].reshape(-1))
            sw.panel.copy_(self.master[o:o + cnt].view(sw.N, sw.Kp))
        self.step_count = int(shards[0]["step"])
        for slot in self._slots.values():
            slot.current_owner = None
        torch.cuda.synchronize()
        if W > 1:
            dist.barrier()

    def materialize(self, model: nn.Module) -> None:
        """Put full weights back into the modules and drop the sharding (for exporting a plain model)."""
        for name, module in model.named_modules():
            sw = getattr(module, "_sharded", None)
            if sw is None:
                continue
            lin = module.base_layer if hasattr(module, "base_layer") else module
            lin.weight.data = sw.full_weight().clone()
            module._sharded = None


def ag_linear(x: torch.Tensor, sw: ShardedWeight) -> torch.Tensor:
    return _AGLinearFn.apply(x, sw, sw.anchor)


def lora_ag_linear(x: torch.Tensor, sw: ShardedWeight, a: torch.Tensor, b: torch.Tensor, scaling: float,
                   residual: torch.Tensor = None, act: str = None) -> torch.Tensor:
    """``act(x W^T + s (x A^T) B^T) + residual`` with ``W`` sharded (``act``: ``None`` or ``"relu_sq"``, never with a
    residual)."""
    return _LoraAGLinearFn.apply(x, sw, a, b, scaling, residual, act)
