"""Batching for pre-shifted ``input_ids`` / ``labels`` datasets.

Collation parity with ``rwkvtune/training/sft_trainer.py:487-546``: truncate to ``ctx_len``, pad to
the longest sample of the batch rounded **up to a multiple of 16**, pad id 0, label pad -100.
Sharding parity with the DistributedSampler Lightning inserts: an epoch permutation seeded by
``seed + epoch``, padded by wrap-around to a multiple of the world size, rank ``r`` takes indices
``r, r + W, ...``; incomplete batches are dropped.  Batches are pinned so the host-to-device copy
can overlap compute, and a small background thread collates ahead of the training loop.
"""
from __future__ import annotations

import queue
import threading
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence

import torch

PAD_MULTIPLE = 16


def collate_batch(samples: Sequence[Dict[str, Any]], ctx_len: int, pad_id: int = 0, pin: bool = True) -> Dict[str, torch.Tensor]:
    ids = [torch.as_tensor(s["input_ids"], dtype=torch.long)[:ctx_len] for s in samples]
    labs = [torch.as_tensor(s["labels"], dtype=torch.long)[:ctx_len] for s in samples]
    width = max(int(t.numel()) for t in ids)
    width = min((width + PAD_MULTIPLE - 1) // PAD_MULTIPLE * PAD_MULTIPLE, max(ctx_len, PAD_MULTIPLE))
    width = (width + PAD_MULTIPLE - 1) // PAD_MULTIPLE * PAD_MULTIPLE
    B = len(ids)
    input_ids = torch.full((B, width), pad_id, dtype=torch.long)
    labels = torch.full((B, width), -100, dtype=torch.long)
    for i, (a, b) in enumerate(zip(ids, labs)):
        input_ids[i, :a.numel()] = a
        labels[i, :b.numel()] = b[:width]
    if pin and torch.cuda.is_available():
        input_ids, labels = input_ids.pin_memory(), labels.pin_memory()
    return {"input_ids": input_ids, "labels": labels}


def epoch_indices(n: int, epoch: int, seed: int, shuffle: bool, rank: int, world: int) -> List[int]:
    if shuffle:
        g = torch.Generator().manual_seed(seed + epoch)
        order = torch.randperm(n, generator=g).tolist()
    else:
        order = list(range(n))
    total = (n + world - 1) // world * world
    order += order[: total - n]
    return order[rank:total:world]


class BatchLoader:
    """Map-style or iterable dataset -> stream of collated, pinned batches for one rank."""

    def __init__(self, dataset, micro_bsz: int, ctx_len: int, rank: int = 0, world: int = 1, shuffle: bool = True,
                 seed: int = 42, prefetch: int = 2, pin: bool = True):
        self.dataset, self.micro_bsz, self.ctx_len = dataset, micro_bsz, ctx_len
        self.rank, self.world, self.shuffle, self.seed = rank, world, shuffle, seed
        self.prefetch, self.pin = prefetch, pin
        self.is_iterable = not hasattr(dataset, "__getitem__") or not hasattr(dataset, "__len__")

    def batches_per_epoch(self) -> Optional[int]:
        if self.is_iterable:
            return None
        per_rank = (len(self.dataset) + self.world - 1) // self.world
        return per_rank // self.micro_bsz

    def _raw_batches(self, epoch: int, skip_batches: int) -> Iterator[List[Dict[str, Any]]]:
        if self.is_iterable:
            buf: List[Dict[str, Any]] = []
            produced = 0
            for i, sample in enumerate(self.dataset):
                if i % self.world != self.rank:
                    continue
                buf.append(sample)
                if len(buf) == self.micro_bsz:
                    if produced >= skip_batches:
                        yield buf
                    produced += 1
                    buf = []
            return
        idx = epoch_indices(len(self.dataset), epoch, self.seed, self.shuffle, self.rank, self.world)
        nb = len(idx) // self.micro_bsz
        for b in range(skip_batches, nb):
            yield [self.dataset[j] for j in idx[b * self.micro_bsz:(b + 1) * self.micro_bsz]]

    def iter_epoch(self, epoch: int, skip_batches: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
        if self.prefetch <= 0:
            for raw in self._raw_batches(epoch, skip_batches):
                yield collate_batch(raw, self.ctx_len, pin=self.pin)
            return
        q: "queue.Queue" = queue.Queue(maxsize=self.prefetch)
        stop = threading.Event()

        def work():
            try:
                for raw in self._raw_batches(epoch, skip_batches):
                    if stop.is_set():
                        return
                    q.put(collate_batch(raw, self.ctx_len, pin=self.pin))
                q.put(None)
            except BaseException as exc:  # surfaced in the consumer
                q.put(exc)

        th = threading.Thread(target=work, daemon=True)
        th.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    return
                if isinstance(item, BaseException):
                    raise item
                yield item
        finally:
            stop.set()
            while not q.empty():
                try:
                    q.get_nowait()
                except queue.Empty:
                    break
