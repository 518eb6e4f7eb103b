"""Fused ZeRO-2 step over peer-mapped (symmetric) memory.

The flat gradient and parameter buffers of every rank are allocated from
``torch.distributed._symmetric_memory`` so that each process holds device pointers to all peers'
buffers.  One optimiser step is then five launches of this repository's own kernels
(``rwkvtune_b200/csrc/zero_p2p.cu``) and no NCCL call:

    barrier -> reduce-scatter + cast/scale + norm partial -> barrier -> clip + AdamW + parameter
    write-back to all ranks (one launch per optimiser group) -> barrier

Device-side waits carry a deadline; the status word is read on the host every ``check_every``
steps (and at checkpoints) so a stuck peer surfaces as a Python exception rather than a hang.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext


class PeerWaitTimeout(RuntimeError):
    pass


def symmetric_allocator(group_name: Optional[str] = None):
    """Returns ``alloc(n, dtype, device)`` producing tensors that can later be rendezvoused."""
    import torch.distributed._symmetric_memory as symm_mem

    def alloc(n: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return symm_mem.empty(n, dtype=dtype, device=device)

    return alloc


def _ptr_array(ptrs: List[int]):
    arr = (ctypes.c_ulonglong * len(ptrs))(*[int(p) for p in ptrs])
    return arr


class FusedZero2:
    def __init__(self, space, ctx, opt, timeout_s: float = 20.0, check_every: int = 50):
        import torch.distributed._symmetric_memory as symm_mem

        self.space, self.ctx, self.opt = space, ctx, opt
        self.W, self.rank = ctx.world_size, ctx.rank
        if space.dtype != torch.bfloat16:
            raise ValueError("the fused ZeRO-2 kernels take bf16 gradients and parameters")
        group = dist.group.WORLD.group_name
        self.ctrl = symm_mem.empty(256, dtype=torch.int32, device=space.device)
        self.ctrl.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        self._h_grads = symm_mem.rendezvous(space.grads, group)
        self._h_params = symm_mem.rendezvous(space.params, group)
        self._h_ctrl = symm_mem.rendezvous(self.ctrl, group)
        self.grad_ptrs = _ptr_array(list(self._h_grads.buffer_ptrs))
        self.param_ptrs = _ptr_array(list(self._h_params.buffer_ptrs))
        self.ctrl_ptrs = _ptr_array(list(self._h_ctrl.buffer_ptrs))
        self.status = torch.zeros(1, dtype=torch.int32, device=space.device)
        self.scratch = torch.zeros(1024, dtype=torch.float32, device=space.device)
        self.gred = torch.empty(opt.hi - opt.lo, dtype=torch.float32, device=space.device)
        self.epoch = 0
        self.timeout_ns = int(timeout_s * 1e9)
        self.check_every = check_every
        self._since_check = 0

    def _barrier(self) -> None:
        self.epoch += 1
        _ext.call("rwkv_p2p_barrier", self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W), _ext.i32(self.epoch),
                  _ext.ptr(self.status), _ext.i64(self.timeout_ns), _ext.stream())

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            raise PeerWaitTimeout(f"rank {self.rank}: device-side wait expired (code {code}: waiting for rank {code % 100})")

    def step(self, lr: float, grad_scale: float = 1.0) -> None:
        opt, sp = self.opt, self.space
        opt.step_count += 1
        self._barrier()                      # every rank's backward has finished writing its gradients
        _ext.call("rwkv_zero2_reduce_scatter", self.grad_ptrs, self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W),
                  _ext.i64(opt.lo), _ext.i64(opt.hi - opt.lo), _ext.f32(grad_scale / self.W), _ext.ptr(self.gred),
                  _ext.ptr(self.scratch), _ext.stream())
        self._barrier()                      # all norm partials published; all peers done reading my gradients
        for gi, s, e in sp.group_segments_in(opt.lo, opt.hi):
            grp = sp.groups[gi]
            a, b = s - opt.lo, e - opt.lo
            _ext.call("rwkv_zero2_adam_broadcast", self.param_ptrs, self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W),
                      _ext.i64(s), _ext.i64(e - s), _ext.ptr(opt.master[a:b]), _ext.ptr(opt.exp_avg[a:b]),
                      _ext.ptr(opt.exp_avg_sq[a:b]), _ext.ptr(self.gred[a:b]), _ext.f32(lr * grp.lr_scale),
                      _ext.f32(opt.beta1), _ext.f32(opt.beta2), _ext.f32(opt.eps), _ext.f32(grp.weight_decay),
                      _ext.i32(opt.step_count), _ext.f32(opt.grad_clip), _ext.stream())
        self._barrier()                      # every rank's parameters are complete before the next forward
        self._since_check += 1
        if self._since_check >= self.check_every:
            self._since_check = 0
            self.check()
