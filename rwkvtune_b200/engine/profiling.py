"""Phase timers, NVTX ranges and an N-step kernel profile for the trainers.

The reference's only tracing aid is ``monitor_memory_and_time`` in its GRPO module
(``rwkvtune/training/grpo/lightning_module.py:34-107``, used around the rollout, reward and
training phases at ``:679``, ``:978``, ``:1347``): wall-clock seconds and allocated / peak device
memory per phase, printed.  :class:`PhaseMonitor` records the same quantities for every phase of
every trainer (forward+backward, reduce+optimiser, prefill, decode, rewards, old log-probs, policy
step), opens an NVTX range per phase so that external timeline tools show them, and hands the
figures to the metric sinks as ``phase/<name>/seconds`` and ``phase/<name>/peak_mem_gb``.

:class:`StepProfiler` wraps the first ``n`` steps after warm-up in ``torch.profiler`` (CUPTI
activity records: no kernel replay, no clock change) and writes the per-kernel device-time table
to ``<proj_dir>/profile_kernels.txt``.  Trainers enable it with ``profile_steps`` in their config or
``RWKVTUNE_PROFILE=<n>`` in the environment.
"""
from __future__ import annotations

import contextlib
import os
import time
from collections import defaultdict
from typing import Dict, Optional

import torch


class PhaseMonitor:
    def __init__(self, device: Optional[torch.device] = None, sync: bool = False, verbose: bool = False):
        self.device = device
        self.cuda = device is not None and device.type == "cuda" and torch.cuda.is_available()
        self.sync = sync            # synchronise at phase boundaries: exact per-phase device time, at the cost of overlap
        self.verbose = verbose
        self.seconds: Dict[str, float] = defaultdict(float)
        self.calls: Dict[str, int] = defaultdict(int)
        self.peak_gb: Dict[str, float] = defaultdict(float)
        self._run_peak = 0          # bytes: peak over the whole run, kept across the per-phase resets below

    def peak_bytes(self) -> int:
        """Peak allocated bytes since this monitor was created.  Phases reset the allocator's own peak counter to
        get a per-phase figure, so the run-wide peak has to be read here, not from ``torch.cuda.max_memory_allocated``."""
        if self.cuda:
            self._run_peak = max(self._run_peak, torch.cuda.max_memory_allocated(self.device))
        return self._run_peak

    @contextlib.contextmanager
    def phase(self, name: str):
        if self.cuda:
            torch.cuda.nvtx.range_push(name)
            if self.sync:
                torch.cuda.synchronize(self.device)
            self.peak_bytes()
            torch.cuda.reset_peak_memory_stats(self.device)
            before = torch.cuda.memory_allocated(self.device)
        t0 = time.perf_counter()
        try:
            yield self
        finally:
            if self.cuda and self.sync:
                torch.cuda.synchronize(self.device)
            dt = time.perf_counter() - t0
            self.seconds[name] += dt
            self.calls[name] += 1
            if self.cuda:
                peak = torch.cuda.max_memory_allocated(self.device) / 2**30
                self.peak_bytes()
                self.peak_gb[name] = max(self.peak_gb[name], peak)
                torch.cuda.nvtx.range_pop()
                if self.verbose:
                    after = torch.cuda.memory_allocated(self.device)
                    print(f"[phase] {name}: {dt:.3f} s, memory {before / 2**30:.2f} -> {after / 2**30:.2f} GB, "
                          f"peak {peak:.2f} GB", flush=True)
            elif self.verbose:
                print(f"[phase] {name}: {dt:.3f} s", flush=True)

    def scalars(self, reset: bool = True) -> Dict[str, float]:
        out = {}
        for name, sec in self.seconds.items():
            out[f"phase/{name}/seconds"] = sec
            if name in self.peak_gb:
                out[f"phase/{name}/peak_mem_gb"] = self.peak_gb[name]
        if reset:
            self.seconds.clear()
            self.calls.clear()
            self.peak_gb.clear()
        return out


def profile_steps_requested(args) -> int:
    env = os.environ.get("RWKVTUNE_PROFILE", "")
    if env.isdigit() and int(env) > 0:
        return int(env)
    return int(getattr(args, "profile_steps", 0) or 0)


class StepProfiler:
    """Profiles steps ``[skip, skip + n)`` of a training loop: call :meth:`step_begin` / :meth:`step_end` around
    each step; the table is written when the last profiled step ends."""

    def __init__(self, n: int, out_dir: str, skip: int = 3, is_main: bool = True, rows: int = 60):
        self.n, self.skip, self.out_dir, self.is_main, self.rows = int(n), skip, out_dir, is_main, rows
        self.seen = 0
        self.prof = None
        self.path = os.path.join(out_dir, "profile_kernels.txt")

    def step_begin(self) -> None:
        if self.n <= 0 or self.prof is not None or self.seen != self.skip:
            return
        from torch.profiler import ProfilerActivity, profile

        acts = [ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(ProfilerActivity.CUDA)
        self.prof = profile(activities=acts)
        self.prof.__enter__()

    def step_end(self) -> None:
        self.seen += 1
        if self.prof is None or self.seen < self.skip + self.n:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.prof.__exit__(None, None, None)
        if self.is_main:
            os.makedirs(self.out_dir, exist_ok=True)
            sort = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
            try:
                table = self.prof.key_averages().table(sort_by=sort, row_limit=self.rows)
            except Exception:
                table = self.prof.key_averages().table(row_limit=self.rows)
            with open(self.path, "w", encoding="utf-8") as fh:
                fh.write(f"{self.n} training steps after {self.skip} warm-up steps\n{table}\n")
            print(f"[profile] kernel table of {self.n} steps written to {self.path}", flush=True)
        self.prof = None
        self.n = 0


def get_gpu_memory_info(device=None) -> Optional[Dict[str, float]]:
    """Allocator figures of one device in GiB (``allocated``, ``reserved``, ``max_allocated``, ``total``,
    ``free`` = total - reserved, ``usage_percent``); ``None`` without CUDA.  Same keys as the reference's
    helper of this name (``rwkvtune/training/grpo/lightning_module.py:34-62``)."""
    if not torch.cuda.is_available():
        return None
    device = torch.cuda.current_device() if device is None else device
    torch.cuda.synchronize(device)
    gib = float(1 << 30)
    total = torch.cuda.get_device_properties(device).total_memory / gib
    reserved = torch.cuda.memory_reserved(device) / gib
    return {"allocated": torch.cuda.memory_allocated(device) / gib, "reserved": reserved,
            "max_allocated": torch.cuda.max_memory_allocated(device) / gib, "total": total, "free": total - reserved,
            "usage_percent": 100.0 * reserved / total if total > 0 else 0.0}


@contextlib.contextmanager
def monitor_memory_and_time(rank, stage_name: str, device=None, sink=print):
    """``with monitor_memory_and_time(rank, "rollout"):`` — one line per use with the wall-clock seconds of the
    block and, on CUDA, the change in allocated memory and the peak inside the block (call convention of
    ``rwkvtune/training/grpo/lightning_module.py:65-107``).  Built on :class:`PhaseMonitor`, so the block also
    shows up as an NVTX range; the monitor is yielded for callers that want the figures instead of the line."""
    dev = None
    if torch.cuda.is_available():
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    mon = PhaseMonitor(dev, sync=True)
    before = get_gpu_memory_info(dev)
    try:
        with mon.phase(stage_name):
            yield mon
    finally:
        stats = mon.scalars(reset=False)
        line = f"[Rank {rank}] {stage_name}: {stats.get(f'phase/{stage_name}/seconds', 0.0):.2f} s"
        after = get_gpu_memory_info(dev)
        if before and after:
            line += (f", allocated {before['allocated']:.2f} -> {after['allocated']:.2f} GiB, "
                     f"peak {stats.get(f'phase/{stage_name}/peak_mem_gb', 0.0):.2f} GiB, "
                     f"reserved {after['reserved']:.2f} of {after['total']:.2f} GiB ({after['usage_percent']:.1f}%)")
        sink(line)
