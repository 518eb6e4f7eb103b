"""Prompt batching for GRPO (``rwkvtune/training/grpo/dataset.py:17-212``).

Each prompt batch is yielded ``repeat_batch_count = steps_per_generation * num_iterations`` times:
the first occurrence triggers a rollout, the following ones consume the buffered slices.  Unlike the
reference, which hands ``rank=0`` to every process so that all ranks read the same shard, each rank
here reads its own shard (``world_size = devices``) and draws with a rank-specific seed.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional

import torch


class RepeatBatchSampler:
    """Yields each batch of indices ``repeat_count`` times in a row.

    Two ways to build it: ``RepeatBatchSampler(n, batch_size, repeat_count, ...)`` draws its own (seeded, rank-sharded)
    permutation of ``range(n)``; ``RepeatBatchSampler(batch_sampler, repeat_batch_count)`` wraps any iterable of index
    batches, which is the reference's form (``rwkvtune/training/grpo/dataset.py:81-124``)."""

    def __init__(self, n, batch_size: Optional[int] = None, repeat_count: int = 1, shuffle: bool = True, seed: int = 42,
                 rank: int = 0, world_size: int = 1, drop_last: bool = True, repeat_batch_count: Optional[int] = None):
        self._wrapped = None if isinstance(n, int) else n
        if repeat_batch_count is not None:
            repeat_count = repeat_batch_count
        elif self._wrapped is not None and batch_size is not None:     # (batch_sampler, repeat_batch_count)
            repeat_count, batch_size = batch_size, None
        if repeat_count <= 0:
            raise ValueError(f"repeat_batch_count must be > 0, got {repeat_count}")
        if self._wrapped is not None:
            batch_size = getattr(self._wrapped, "batch_size", batch_size)
            drop_last = bool(getattr(self._wrapped, "drop_last", False))
            n = 0
        elif batch_size is None:
            raise ValueError("batch_size is required")
        self.n, self.batch_size, self.repeat_count = n, batch_size, repeat_count
        self.shuffle, self.seed, self.rank, self.world_size, self.drop_last = shuffle, seed, rank, world_size, drop_last
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch
        inner = getattr(self._wrapped, "sampler", None)
        if inner is not None and hasattr(inner, "set_epoch"):
            inner.set_epoch(epoch)

    @property
    def sampler(self):
        """The index source behind the batches (this object itself when it draws its own permutation)."""
        return self if self._wrapped is None else getattr(self._wrapped, "sampler", None)

    def _indices(self) -> List[int]:
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            order = torch.randperm(self.n, generator=g).tolist()
        else:
            order = list(range(self.n))
        total = (self.n + self.world_size - 1) // self.world_size * self.world_size
        order += order[: total - self.n]
        return order[self.rank:total:self.world_size]

    def num_batches(self) -> int:
        if self._wrapped is not None:
            return len(self._wrapped)
        per_rank = (self.n + self.world_size - 1) // self.world_size
        return per_rank // self.batch_size if self.drop_last else -(-per_rank // self.batch_size)

    def __len__(self) -> int:
        return self.num_batches() * self.repeat_count

    def __iter__(self) -> Iterator[List[int]]:
        if self._wrapped is not None:
            for batch in self._wrapped:
                for _ in range(self.repeat_count):
                    yield batch
            return
        idx = self._indices()
        for b in range(self.num_batches()):
            batch = idx[b * self.batch_size:(b + 1) * self.batch_size]
            for _ in range(self.repeat_count):
                yield batch


def grpo_collate(samples: List[Dict[str, Any]]) -> Dict[str, Any]:
    """``{"prompts": [...], "input_ids": [[...], ...], <every other column>: [...]}``."""
    out: Dict[str, Any] = {"prompts": [s["prompt"] for s in samples],
                           "input_ids": [list(s["input_ids"]) for s in samples]}
    for key in samples[0]:
        if key not in ("prompt", "input_ids"):
            out[key] = [s[key] for s in samples]
    return out


class GRPODataLoader:
    def __init__(self, dataset, sampler: RepeatBatchSampler):
        self.dataset, self.sampler = dataset, sampler

    def __len__(self) -> int:
        return len(self.sampler)

    def __iter__(self):
        for idx in self.sampler:
            yield grpo_collate([self.dataset[i] for i in idx])


def create_grpo_dataloader(dataset, batch_size: int, repeat_batch_count: int = 1, shuffle: bool = True, seed: int = 42,
                           rank: int = 0, world_size: int = 1, num_workers: int = 0) -> GRPODataLoader:
    first = dataset[0]
    for col in ("prompt", "input_ids"):
        if col not in first:
            raise ValueError(f"GRPO dataset samples need a {col!r} field")
    return GRPODataLoader(dataset, RepeatBatchSampler(len(dataset), batch_size, repeat_batch_count, shuffle, seed, rank,
                                                      world_size))


class GRPODataBuffer:
    """Bounded FIFO of rollout samples (``rwkvtune/training/grpo/dataset.py:17-78``).

    ``add_batch`` splits a rollout of ``B*G`` completions into per-sample records, ``sample_batch`` draws a random
    training batch of stacked tensors.  ``add`` / ``pop`` move whole slices (what the trainer itself uses)."""

    _TENSOR_FIELDS = ("prompt_ids", "completion_ids", "completion_logps", "rewards", "advantages", "masks")

    def __init__(self, buffer_size: int = 1000, capacity: Optional[int] = None):
        from collections import deque

        self.buffer_size = int(capacity if capacity is not None else buffer_size)
        self.buffer = deque(maxlen=self.buffer_size)

    # reference-style per-sample interface ---------------------------------------------------------------------
    def add_batch(self, prompts, prompt_ids, completions, completion_ids, completion_logps, rewards, advantages,
                  masks) -> None:
        cols = (prompt_ids, completion_ids, completion_logps, rewards, advantages, masks)
        for i, (prompt, completion) in enumerate(zip(prompts, completions)):
            record = {"prompt": prompt, "completion": completion}
            record.update({name: col[i] for name, col in zip(self._TENSOR_FIELDS, cols)})
            self.buffer.append(record)

    def sample_batch(self, batch_size: int, generator: Optional[torch.Generator] = None):
        """Random batch without replacement (``None`` when the buffer is empty)."""
        if not self.buffer:
            return None
        picks = torch.randperm(len(self.buffer), generator=generator)[:batch_size].tolist()
        rows = [self.buffer[i] for i in picks]
        return {name: torch.stack([row[name] for row in rows]) for name in self._TENSOR_FIELDS}

    def is_full(self) -> bool:
        return len(self.buffer) >= self.buffer_size

    # slice interface ------------------------------------------------------------------------------------------
    @property
    def capacity(self) -> int:
        return self.buffer_size

    @property
    def items(self):
        return self.buffer

    def add(self, item) -> None:
        self.buffer.append(item)

    def pop(self):
        return self.buffer.popleft() if self.buffer else None

    def __len__(self) -> int:
        return len(self.buffer)

    def clear(self) -> None:
        self.buffer.clear()
