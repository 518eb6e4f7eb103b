"""Flat parameter space: every trainable parameter is a view into one contiguous buffer.

Optimiser state sharding (ZeRO) then reduces to offset arithmetic on ``[0, numel)``:
rank ``r`` of ``W`` owns ``[r * shard, (r + 1) * shard)`` where ``shard = padded / W``.
Because ownership is a pure function of (offset, world size), a checkpoint written with
one world size can be re-sharded for another without touching the tensors' contents.

Parameters are ordered by optimiser group so that each group is one contiguous range and
the fused AdamW kernel runs once per (group ∩ shard) segment.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

ALIGN = 128  # elements; keeps every segment 256-byte aligned in bf16


@dataclass
class ParamGroupSpec:
    name: str
    lr_scale: float = 1.0
    weight_decay: float = 0.0
    params: List[Tuple[str, torch.nn.Parameter]] = field(default_factory=list)


@dataclass
class Segment:
    name: str
    start: int
    numel: int
    shape: Tuple[int, ...]
    group: int


class FlatParamSpace:
    def __init__(self, groups: Sequence[ParamGroupSpec], world_size: int = 1, dtype: torch.dtype = None,
                 device: torch.device = None, allocator: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None):
        params = [p for g in groups for _, p in g.params]
        if not params:
            raise ValueError("no trainable parameters")
        self.dtype = dtype or params[0].dtype
        self.device = device or params[0].device
        self.world_size = world_size
        self.groups = list(groups)
        self.segments: List[Segment] = []
        self.group_ranges: List[Tuple[int, int]] = []
        off = 0
        for gi, g in enumerate(groups):
            g_start = off
            for name, p in g.params:
                self.segments.append(Segment(name, off, p.numel(), tuple(p.shape), gi))
                off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            self.group_ranges.append((g_start, off))
        self.numel = off
        quantum = ALIGN * world_size
        self.padded = (off + quantum - 1) // quantum * quantum
        self.shard_numel = self.padded // world_size
        alloc = allocator or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
        self.params = alloc(self.padded, self.dtype, self.device)
        self.grads = alloc(self.padded, self.dtype, self.device)
        self.params.zero_()
        self.grads.zero_()
        with torch.no_grad():
            for seg, p in zip(self.segments, params):
                view = self.params[seg.start:seg.start + seg.numel].view(seg.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.grads[seg.start:seg.start + seg.numel].view(seg.shape)
        self._params_list = params

    def shard_range(self, rank: int) -> Tuple[int, int]:
        return rank * self.shard_numel, (rank + 1) * self.shard_numel

    def rebind_grads(self) -> None:
        """Re-attach ``.grad`` views (needed after something set ``p.grad = None``)."""
        for seg, p in zip(self.segments, self._params_list):
            p.grad = self.grads[seg.start:seg.start + seg.numel].view(seg.shape)

    def zero_grads(self) -> None:
        self.grads.zero_()

    def group_segments_in(self, lo: int, hi: int) -> List[Tuple[int, int, int]]:
        """Intersections of ``[lo, hi)`` with each group's range: ``(group_index, start, end)``."""
        out = []
        for gi, (gs, ge) in enumerate(self.group_ranges):
            s, e = max(lo, gs), min(hi, ge)
            if s < e:
                out.append((gi, s, e))
        if hi > self.numel and lo < hi:   # padding tail belongs to the last group (all zeros)
            pass
        return out

    def named_views(self) -> Iterable[Tuple[str, torch.Tensor]]:
        for seg in self.segments:
            yield seg.name, self.params[seg.start:seg.start + seg.numel].view(seg.shape)


def build_param_groups(named_params: Iterable[Tuple[str, torch.nn.Parameter]], weight_decay: float,
                       lr_2x_patterns: Sequence[str] = (), decay_filter: Optional[Callable[[str, torch.nn.Parameter], bool]] = None
                       ) -> List[ParamGroupSpec]:
    """Optimiser grouping of the reference.

    Weight decay applies to parameters with ``ndim >= 2`` whose name contains ``.weight`` (when
    ``weight_decay > 0``); names matching ``lr_2x_patterns`` get twice the learning rate
    (``att.w0`` in the infinite-context and GRPO modules:
    ``rwkvtune/training/lightning_module_infctx.py:479-487``).  The standard SFT/pretrain module's
    patterns (``time_first`` ...) match nothing in RWKV-7, so it passes no patterns
    (``rwkvtune/training/lightning_module.py:234-246``).
    """
    g1 = ParamGroupSpec("lr_1x", 1.0, 0.0)
    g2 = ParamGroupSpec("lr_2x", 2.0, 0.0)
    gd = ParamGroupSpec("decay", 1.0, weight_decay)
    for name, p in named_params:
        if not p.requires_grad:
            continue
        if any(pat in name for pat in lr_2x_patterns):
            g2.params.append((name, p))
        elif weight_decay > 0 and (decay_filter(name, p) if decay_filter else (p.ndim >= 2 and ".weight" in name)):
            gd.params.append((name, p))
        else:
            g1.params.append((name, p))
    return [g for g in (g1, g2, gd) if g.params]
