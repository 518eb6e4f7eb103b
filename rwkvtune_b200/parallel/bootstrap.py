"""Process-group bootstrap: one process per GPU, NCCL on CUDA and gloo on CPU.

The reference lets PyTorch Lightning create the default process group
(``rwkvtune/training/sft_trainer.py:440-446``); here the launcher environment
(``RANK``/``LOCAL_RANK``/``WORLD_SIZE``/``MASTER_ADDR``/``MASTER_PORT``) is read directly.
A second, gloo-backed group is created next to NCCL for host-side votes and timeouts.
"""
from __future__ import annotations

import atexit
import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistContext:
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    device: torch.device = torch.device("cpu")
    backend: str = "none"
    control_group: Optional[object] = None   # gloo group for CPU-side coordination

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier()

    def all_agree(self, ok: bool) -> bool:
        """True only if every rank passed ``ok=True``.  A host-side MIN-reduction: it runs on the gloo control
        group when there is one, so it neither launches a kernel nor waits for the GPU."""
        if self.world_size <= 1:
            return bool(ok)
        if self.control_group is not None:
            t = torch.tensor([1 if ok else 0], dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.control_group)
        else:
            t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(int(t.item()))

    def store(self):
        """The rendezvous key-value store of the default process group (None in single-process runs)."""
        if self.world_size <= 1 or not dist.is_initialized():
            return None
        from torch.distributed import distributed_c10d

        return distributed_c10d._get_default_store()


def env_world() -> tuple:
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


def init_distributed(accelerator: str = "auto", timeout_s: float = 600.0) -> DistContext:
    """Initialise (or adopt) the default process group and select this rank's device."""
    rank, local_rank, world = env_world()
    use_cuda = accelerator in ("gpu", "cuda", "auto") and torch.cuda.is_available()
    if accelerator in ("gpu", "cuda") and not torch.cuda.is_available():
        raise RuntimeError("accelerator='gpu' requested but no CUDA device is visible")
    device = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    ctx = DistContext(rank, local_rank, world, device, "none")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = "nccl" if use_cuda else "gloo"
        if not dist.is_initialized():
            kwargs = {"device_id": device} if use_cuda else {}
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
            if backend == "gloo":
                # A process that exits with a live gloo group can die in its C++ teardown ("terminate called without
                # an active exception": about one 8-rank run in four here), which turns a finished run into a failed
                # one.  Destroying a gloo group is local - no peer takes part - so it is safe on every way out.
                atexit.register(_shutdown_quietly)
        ctx.backend = dist.get_backend()
        if ctx.backend == "nccl":
            ctx.control_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    return ctx


def shutdown() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def _shutdown_quietly() -> None:
    try:
        shutdown()
    except Exception:      # interpreter is going down; a failed teardown must not replace the real exit status
        pass
