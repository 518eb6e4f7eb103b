"""Fused ZeRO-2 step over peer-mapped (symmetric) memory, with the gradient reduce-scatter overlapped with backward.

The flat gradient and parameter buffers of every rank are allocated from
``torch.distributed._symmetric_memory`` so that each process holds device pointers to all peers'
buffers.  The flat gradient space is cut into *buckets* of whole parameters.  During backward a
post-accumulate hook counts down the parameters of each bucket; when a bucket's last gradient has
been written the rank

1. raises the bucket's flag in every peer's control block (one tiny kernel on the compute stream),
2. and, if part of the bucket lies in the range this rank owns, queues on a side stream a bounded wait
   for all ranks' flags of that bucket followed by the reduce kernel for that range (peer loads of all
   ranks' gradients in fixed rank order, bf16 -> fp32, scale, optional fp32 accumulation over
   micro-batches, squared-norm partial),

while backward goes on with the next layers.  The optimiser step then only has to flush buckets
whose parameters received no gradient, join the side stream, publish the squared-norm share,
meet the peers at a flag barrier, and run clip + AdamW + write-back of the new bf16 parameters into
every rank's parameter buffer (one launch per optimiser group), followed by a closing barrier.  All of
it is this repository's own kernels (``rwkvtune_b200/csrc/zero_p2p.cu``); no NCCL call is on the path.
It does the job of DeepSpeed's stage-2 ``overlap_comm`` reduce-scatter, FusedAdam and parameter
all-gather that the reference selects by ``strategy="deepspeed_stage_2"``
(``rwkvtune/training/sft_trainer.py:392-412``).

Every device-side wait carries a deadline.  When one expires the kernel records a code in the
status word and every later data kernel of the step returns without writing (the parameters keep
their previous values); the status word is copied to pinned host memory at the end of each step and
``check()`` reads that copy without a device synchronisation, so the host sees a stuck peer at the
next step boundary.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext

MAX_BUCKETS = 1024
BUCKET_WORD0 = 128            # first bucket flag word of the control block
CTRL_WORDS = BUCKET_WORD0 + 16 * MAX_BUCKETS
REDUCE_BLOCKS = 1024


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


def plan_buckets(segments, padded: int, bucket_numel: int, max_buckets: int = MAX_BUCKETS):
    """Cut the flat space ``[0, padded)`` into buckets of whole parameters.

    ``segments``: ``[(start, numel), ...]`` in flat order.  Returns ``(bounds, seg_bucket)`` where bucket ``b``
    covers ``[bounds[b], bounds[b + 1])`` and ``seg_bucket[i]`` is the bucket of segment ``i``.  A bucket closes as
    soon as it holds at least ``bucket_numel`` elements; the tail padding belongs to the last bucket."""
    total = sum(n for _, n in segments)
    bucket_numel = max(int(bucket_numel), -(-total // max_buckets), 1)
    bounds, seg_bucket = [0], []
    filled = 0
    for i, (start, numel) in enumerate(segments):
        seg_bucket.append(len(bounds) - 1)
        filled += numel
        nxt = segments[i + 1][0] if i + 1 < len(segments) else padded
        if filled >= bucket_numel and i + 1 < len(segments):
            bounds.append(nxt)
            filled = 0
    bounds.append(padded)
    return bounds, seg_bucket


class FusedZero2:
    def __init__(self, space, ctx, opt, timeout_s: float = 20.0, bucket_mb: float = 64.0):
        import torch.distributed._symmetric_memory as symm_mem

        self.space, self.ctx, self.opt = space, ctx, opt
        self.W, self.rank = ctx.world_size, ctx.rank
        if space.dtype != torch.bfloat16:
            raise ValueError("the fused ZeRO-2 kernels take bf16 gradients and parameters")
        dev = space.device
        group = dist.group.WORLD.group_name
        self.ctrl = symm_mem.empty(CTRL_WORDS, dtype=torch.int32, device=dev)
        self.ctrl.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        self._h_grads = symm_mem.rendezvous(space.grads, group)
        self._h_params = symm_mem.rendezvous(space.params, group)
        self._h_ctrl = symm_mem.rendezvous(self.ctrl, group)
        self.grad_ptrs = _ptr_array(list(self._h_grads.buffer_ptrs))
        self.param_ptrs = _ptr_array(list(self._h_params.buffer_ptrs))
        self.ctrl_ptrs = _ptr_array(list(self._h_ctrl.buffer_ptrs))
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.gred = torch.zeros(opt.hi - opt.lo, dtype=torch.float32, device=dev)
        self.epoch = 0
        self.timeout_ns = int(timeout_s * 1e9)
        self.overlap = True

        # ---- buckets of whole parameters and this rank's reduce launches
        segs = [(s.start, s.numel) for s in space.segments]
        self.bounds, self.seg_bucket = plan_buckets(segs, space.padded, int(bucket_mb * (1 << 20)) // 2)
        self.n_buckets = len(self.bounds) - 1
        self.bucket_params = [0] * self.n_buckets
        for b in self.seg_bucket:
            self.bucket_params[b] += 1
        self.launch_of_bucket = {}      # bucket -> (slot, lo, n) : the part of the bucket inside the owned range
        for b in range(self.n_buckets):
            lo, hi = max(self.bounds[b], opt.lo), min(self.bounds[b + 1], opt.hi)
            if lo < hi:
                self.launch_of_bucket[b] = (len(self.launch_of_bucket), lo, hi - lo)
        self.partials = torch.zeros(max(1, len(self.launch_of_bucket)) * REDUCE_BLOCKS, dtype=torch.float32, device=dev)
        self.extra_sumsq: Optional[torch.Tensor] = None   # squared norm of gradients reduced elsewhere (ZeRO-3 panels)
        self.before_publish = None    # callable(): runs before this rank's norm share is published
        self.after_norm = None        # callable(lr): runs once every rank's norm share has arrived
        self.comm = torch.cuda.Stream(device=dev)
        self._events = [torch.cuda.Event() for _ in range(self.n_buckets)]
        self._joined = torch.cuda.Event()
        self._pending = list(self.bucket_params)
        self._signalled = [False] * self.n_buckets
        self._armed = False
        self._micro = 0            # micro-batches reduced since the last optimiser step
        self._in_flight = False    # True between the first signal of a micro-batch and its finish
        self.flag_epoch = 0
        self.timing = None         # set to a list to collect (backward done, step done) CUDA event pairs per step
        self._t0 = None
        self._hooks = []
        for i, p in enumerate(space._params_list):
            self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(self.seg_bucket[i])))

    # ------------------------------------------------------------------ flag helpers
    def _barrier(self) -> None:
        self.epoch += 1
        _ext.call("rwkv_p2p_barrier", self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W), _ext.i32(self.epoch),
                  _ext.ptr(self.status), _ext.i64(self.timeout_ns), _ext.stream())

    def check(self) -> None:
        """Raise if a device-side wait expired during a finished step (reads the pinned host copy of the status
        word, which the end of every step refreshes: no device synchronisation)."""
        code = int(self.status_host[0])
        if code:
            raise PeerWaitTimeout(f"rank {self.rank}: device-side wait expired (code {code}: waiting for rank {code % 100})")

    def check_now(self) -> None:
        """Same, reading the device word directly (synchronises)."""
        code = int(self.status.item())
        if code:
            raise PeerWaitTimeout(f"rank {self.rank}: device-side wait expired (code {code}: waiting for rank {code % 100})")

    # ------------------------------------------------------------------ bucket pipeline
    def _make_hook(self, bucket: int):
        def hook(_param):
            if not self._armed:
                return
            self._pending[bucket] -= 1
            if self._pending[bucket] == 0:
                self._bucket_ready(bucket)

        return hook

    def arm(self, grad_scale: float = 1.0) -> None:
        """Call before the backward pass of a micro-batch: buckets are reduced as their gradients complete.  Only
        for a backward pass that produces every parameter's gradient exactly once (not for chunked back-propagation
        through time, where a parameter receives one gradient per chunk)."""
        if not self.overlap:
            return
        self._scale = grad_scale / self.W
        self._pending = list(self.bucket_params)
        self._signalled = [False] * self.n_buckets
        self._armed = True
        self.flag_epoch += 1
        self._in_flight = True

    def _bucket_ready(self, b: int) -> None:
        """The last gradient of bucket ``b`` has been queued on the current stream."""
        self._signalled[b] = True
        st = _ext.stream()
        word = BUCKET_WORD0 + 16 * b
        _ext.call("rwkv_p2p_signal", self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W), _ext.i32(word),
                  _ext.i32(self.flag_epoch), st)
        launch = self.launch_of_bucket.get(b)
        if launch is None:
            return
        slot, lo, n = launch
        ev = self._events[b]
        ev.record(torch.cuda.current_stream())
        self.comm.wait_event(ev)
        cst = ctypes.c_void_p(self.comm.cuda_stream)
        _ext.call("rwkv_p2p_wait", self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W), _ext.i32(word),
                  _ext.i32(self.flag_epoch), _ext.ptr(self.status), _ext.i64(self.timeout_ns), cst)
        blocks = max(1, min(REDUCE_BLOCKS, (n // 8 + 255) // 256))
        part = self.partials[slot * REDUCE_BLOCKS:(slot + 1) * REDUCE_BLOCKS]   # entries past `blocks` stay zero
        _ext.call("rwkv_zero2_reduce_bucket", self.grad_ptrs, _ext.i32(self.W), _ext.i64(lo), _ext.i64(n),
                  _ext.f32(self._scale), _ext.ptr(self.gred[lo - self.opt.lo:]), _ext.ptr(part), _ext.i32(blocks),
                  _ext.i32(1 if self._micro > 0 else 0), _ext.ptr(self.status), cst)

    _scale = 1.0

    def finish_micro(self, boundary: bool, grad_scale: float = 1.0) -> None:
        """Call after the backward pass of a micro-batch.  Buckets that were not reduced during backward (hooks not
        armed, parameters without a gradient) are flushed now.  On a non-boundary micro-batch the ranks then meet so
        that every owner has read this micro-batch's gradients, and the local gradient buffer is cleared for the
        next one (the fp32 sum lives in the owner's reduced shard)."""
        if self.timing is not None and boundary:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        if not self._in_flight:          # hooks were not armed: everything goes out now
            self._pending = list(self.bucket_params)
            self._signalled = [False] * self.n_buckets
            self.flag_epoch += 1
            self._scale = grad_scale / self.W
        self._armed = False
        for b in range(self.n_buckets):
            if not self._signalled[b]:
                self._bucket_ready(b)
        self._in_flight = False
        self._micro += 1
        self._joined.record(self.comm)
        torch.cuda.current_stream().wait_event(self._joined)
        if not boundary:
            self._barrier()              # every owner has consumed this micro-batch's gradients
            self.space.grads.zero_()

    def step(self, lr: float, grad_scale: float = 1.0) -> None:
        opt, sp = self.opt, self.space
        if self._micro == 0 or self._in_flight:    # caller did not go through finish_micro
            self.finish_micro(True, grad_scale)
        opt.step_count += 1
        n_part = len(self.launch_of_bucket) * REDUCE_BLOCKS
        if self.before_publish is not None:
            self.before_publish()
        _ext.call("rwkv_zero2_publish_norm", _ext.ptr(self.partials), _ext.i32(n_part), _ext.ptr(self.extra_sumsq),
                  self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W), _ext.stream())
        self._barrier()                      # all norm shares published; all peers done reading my gradients
        if self.after_norm is not None:
            self.after_norm(lr)
        for gi, s, e in sp.group_segments_in(opt.lo, opt.hi):
            grp = sp.groups[gi]
            a, b = s - opt.lo, e - opt.lo
            _ext.call("rwkv_zero2_adam_broadcast", self.param_ptrs, self.ctrl_ptrs, _ext.i32(self.rank), _ext.i32(self.W),
                      _ext.i64(s), _ext.i64(e - s), _ext.ptr(opt.master[a:b]), _ext.ptr(opt.exp_avg[a:b]),
                      _ext.ptr(opt.exp_avg_sq[a:b]), _ext.ptr(self.gred[a:b]), _ext.f32(lr * grp.lr_scale),
                      _ext.f32(opt.beta1), _ext.f32(opt.beta2), _ext.f32(opt.eps), _ext.f32(grp.weight_decay),
                      _ext.i32(opt.step_count), _ext.f32(opt.grad_clip), _ext.ptr(self.status), _ext.stream())
        self._barrier()                      # every rank's parameters are complete before the next forward
        self.status_host.copy_(self.status, non_blocking=True)
        self._micro = 0
        if self.timing is not None and self._t0 is not None:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record()
            self.timing.append((self._t0, t1))
            self._t0 = None
