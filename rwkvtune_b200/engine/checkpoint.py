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
    zero3 = getattr(engine, "zero3", None)
    if save_optimizer and zero3 is not None and zero3.trainable:   # optimiser state of the K-panels this rank owns
        torch.save(zero3.state_dict(), os.path.join(sdir, f"panels{ctx.rank}.pt"))
    if ctx.rank == 0:
        meta = {"format": 1, "time": time.time(), "world_size": ctx.world_size, "stage": opt.stage,
                "optimizer_steps": engine.optimizer_steps, "micro_step": engine.micro_step,
                "tokens_seen": engine.tokens_seen, "numel": engine.space.numel, "has_optimizer": bool(save_optimizer),
                "segments": [[s.name, s.start, s.numel] for s in engine.space.segments]}
        meta.update(extra_meta)
        with open(os.path.join(sdir, META), "w", encoding="utf-8") as fh:
            json.dump(meta, fh, indent=1)


def atomic_checkpoint(final_dir: str, ctx, write_fn) -> None:
    """Run ``write_fn(tmp_dir)`` on every rank, then publish ``tmp_dir`` as ``final_dir``.

    The directory is published only if **every** rank wrote its part: the ranks agree on a success flag
    (a host-side MIN-reduction) between the writes and the rename, so a rank that failed to write its optimiser
    shard (disk full, I/O error) vetoes the checkpoint instead of leaving one with a missing shard.  An existing
    ``final_dir`` is renamed aside first and deleted only after the new one is in place; on a veto the temporary
    directory is removed, the old checkpoint stays, and every rank raises."""
    tmp = final_dir + ".tmp"
    old = final_dir + ".old"
    if ctx.rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
        os.makedirs(tmp, exist_ok=True)
    _barrier(ctx)
    error: Optional[BaseException] = None
    try:
        write_fn(tmp)
    except Exception as exc:   # the other ranks must still reach the agreement below
        error = exc
    everyone_ok = ctx.all_agree(error is None)
    if ctx.rank == 0:
        if everyone_ok:
            shutil.rmtree(old, ignore_errors=True)
            if os.path.exists(final_dir):
                os.replace(final_dir, old)
            os.replace(tmp, final_dir)
            shutil.rmtree(old, ignore_errors=True)
        else:
            shutil.rmtree(tmp, ignore_errors=True)
    _barrier(ctx)
    if error is not None:
        raise error
    if not everyone_ok:
        raise RuntimeError(f"checkpoint {final_dir} was not published: another rank failed to write its part")


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


def check_shards(shards: List[Dict[str, Any]], where: str = "") -> None:
    """A sharded optimiser state is usable only if every rank's file is there and the owned ranges tile the flat
    space without gaps: one file per saved rank, ``lo`` of each shard equal to ``hi`` of the previous one."""
    world = int(shards[0]["world_size"])
    if len(shards) != world:
        raise RuntimeError(f"{where}: optimiser state was saved by {world} ranks but {len(shards)} shard files exist")
    ordered = sorted(shards, key=lambda s: s["lo"])
    pos = 0
    for s in ordered:
        if int(s["lo"]) != pos:
            raise RuntimeError(f"{where}: optimiser shards do not tile the parameter space (gap or overlap at {pos})")
        pos = int(s["hi"])
    if pos != int(ordered[0]["padded"]):
        raise RuntimeError(f"{where}: optimiser shards end at {pos}, expected {ordered[0]['padded']}")


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
    try:
        shards = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    except Exception as exc:   # truncated or corrupt shard: fall back to a weights-only resume, loudly
        if ctx.is_main:
            print(f"[checkpoint] optimiser state under {ckpt_dir} is unreadable ({type(exc).__name__}: {exc}); "
                  "resuming from the weights only")
        return False
    if shards[0]["stage"] == 0:
        shards = shards[:1]
    else:
        check_shards(shards, ckpt_dir)
    master, m, v, step = merge_shards(shards)
    dev = engine.space.device
    engine.opt.load_full_state(master.to(dev), m.to(dev), v.to(dev), step)
    zero3 = getattr(engine, "zero3", None)
    if zero3 is not None and zero3.trainable:
        pfiles = sorted(glob.glob(os.path.join(ckpt_dir, STATE_DIR, "panels*.pt")))
        if pfiles:
            zero3.load_state([torch.load(f, map_location="cpu", weights_only=False) for f in pfiles])
    engine.optimizer_steps = int(meta.get("optimizer_steps", step))
    engine.micro_step = int(meta.get("micro_step", 0))
    engine.tokens_seen = int(meta.get("tokens_seen", 0))
    return True
