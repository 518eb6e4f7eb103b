"""Trainer-state checkpoints: crash-safe writes, rotation, and resume across world sizes.

A save point is a directory ``<proj_dir>/rwkv7-{epoch|batch}{N}/`` holding the hub-format model (or
adapter) files written by :mod:`rwkvtune_b200.training.model_save_utils` plus ``trainer_state/``:

    meta.json        step counters, samples_seen, world geometry, LR position, RNG seeds
    rank{r}.pt       this rank's slice of the flat fp32 master weights and Adam moments

The directory is first written as ``<name>.tmp``, all ranks meet at a barrier, rank 0 renames it
into place and the ranks meet again, so a crash leaves either the old state or the complete new
one (same protocol as ``rwkvtune/training/callbacks.py:337-370``).  Because optimiser ownership is a
contiguous range of one flat vector (:class:`FlatParamSpace`), loading with a different number of
ranks concatenates the shards and re-slices them: the reference's elastic mode restores weights
only (``rwkvtune/training/sft_trainer.py:705-723``), this one keeps the optimiser state.
"""
from __future__ import annotations

import glob
import json
import os
import shutil
import time
from typing import Any, Dict, List, Optional

import torch

from ..parallel.zero import merge_shards

STATE_DIR = "trainer_state"
META = "meta.json"


def _barrier(ctx) -> None:
    if ctx.world_size > 1:
        ctx.barrier()


def save_trainer_state(dirpath: str, engine, ctx, extra_meta: Dict[str, Any], save_optimizer: bool = True) -> None:
    """Write ``trainer_state/`` inside an existing (temporary) checkpoint directory."""
    sdir = os.path.join(dirpath, STATE_DIR)
    os.makedirs(sdir, exist_ok=True)
    opt = engine.opt
    if save_optimizer and (opt.stage >= 1 or ctx.rank == 0):
        torch.save(opt.state_dict(), os.path.join(sdir, f"rank{ctx.rank}.pt"))
    if ctx.rank == 0:
        meta = {"format": 1, "time": time.time(), "world_size": ctx.world_size, "stage": opt.stage,
                "optimizer_steps": engine.optimizer_steps, "micro_step": engine.micro_step,
                "tokens_seen": engine.tokens_seen, "numel": engine.space.numel, "has_optimizer": bool(save_optimizer),
                "segments": [[s.name, s.start, s.numel] for s in engine.space.segments]}
        meta.update(extra_meta)
        with open(os.path.join(sdir, META), "w", encoding="utf-8") as fh:
            json.dump(meta, fh, indent=1)


def atomic_checkpoint(final_dir: str, ctx, write_fn) -> None:
    """Run ``write_fn(tmp_dir)`` on every rank, then publish ``tmp_dir`` as ``final_dir`` atomically."""
    tmp = final_dir + ".tmp"
    if ctx.rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
        os.makedirs(tmp, exist_ok=True)
    _barrier(ctx)
    ok = True
    try:
        write_fn(tmp)
    except Exception:
        ok = False
        raise
    finally:
        _barrier(ctx)   # reached on failure too, so the other ranks do not hang
        if ok and ctx.rank == 0:
            shutil.rmtree(final_dir, ignore_errors=True)
            os.replace(tmp, final_dir)
        _barrier(ctx)


def rotate_checkpoints(proj_dir: str, keep: int, pattern: str = "rwkv7-*") -> List[str]:
    """Delete all but the ``keep`` newest checkpoint directories; returns what was removed."""
    if keep <= 0:
        return []
    dirs = [d for d in glob.glob(os.path.join(proj_dir, pattern)) if os.path.isdir(d) and not d.endswith(".tmp")]
    dirs.sort(key=os.path.getmtime)
    doomed = dirs[:-keep] if len(dirs) > keep else []
    for d in doomed:
        shutil.rmtree(d, ignore_errors=True)
    return doomed


def find_checkpoint(path: str) -> Optional[str]:
    """Resolve ``resume_from_checkpoint``: a checkpoint directory, a parent directory (newest child with
    a trainer state wins) or ``"latest"`` handled by the caller."""
    if path is None:
        return None
    if os.path.isdir(os.path.join(path, STATE_DIR)) or os.path.exists(os.path.join(path, "model.pth")) \
            or os.path.exists(os.path.join(path, "adapter_model.bin")):
        return path
    if os.path.isdir(path):
        cands = [d for d in glob.glob(os.path.join(path, "*")) if os.path.isdir(os.path.join(d, STATE_DIR))]
        if cands:
            return max(cands, key=os.path.getmtime)
    if os.path.isfile(path):
        return path
    return None


def read_meta(ckpt_dir: str) -> Dict[str, Any]:
    p = os.path.join(ckpt_dir, STATE_DIR, META)
    if not os.path.exists(p):
        return {}
    with open(p, "r", encoding="utf-8") as fh:
        return json.load(fh)


def load_optimizer_state(ckpt_dir: str, engine, ctx) -> bool:
    """Restore master weights and Adam moments, re-sharding if the world size changed."""
    meta = read_meta(ckpt_dir)
    if not meta.get("has_optimizer"):
        return False
    if meta.get("numel") != engine.space.numel or [s[0] for s in meta.get("segments", [])] != [s.name for s in engine.space.segments]:
        return False   # different trainable set: weights-only resume
    files = sorted(glob.glob(os.path.join(ckpt_dir, STATE_DIR, "rank*.pt")),
                   key=lambda f: int(os.path.basename(f)[4:-3]))
    if not files:
        return False
    shards = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    if shards[0]["stage"] == 0:
        shards = shards[:1]
    master, m, v, step = merge_shards(shards)
    dev = engine.space.device
    engine.opt.load_full_state(master.to(dev), m.to(dev), v.to(dev), step)
    engine.optimizer_steps = int(meta.get("optimizer_steps", step))
    engine.micro_step = int(meta.get("micro_step", 0))
    engine.tokens_seen = int(meta.get("tokens_seen", 0))
    return True
