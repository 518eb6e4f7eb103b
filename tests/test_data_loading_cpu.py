"""Batch loading: collation (truncate to ctx_len, pad to a multiple of 16, pad id 0 / label -100), the per-rank split,
epoch shuffling, skipping on resume, iterable datasets and errors raised inside the prefetch thread."""
import pytest
import torch

from rwkvtune_b200.training.data_loading import BatchLoader, collate_batch, epoch_indices


def _rows(n, lengths=None):
    lengths = lengths or [10] * n
    return [{"input_ids": list(range(100 * i + 1, 100 * i + 1 + L)), "labels": list(range(100 * i + 2, 100 * i + 2 + L))}
            for i, L in enumerate(lengths)]


def test_collation_truncates_pads_to_sixteen_and_masks_padding():
    batch = collate_batch(_rows(3, [5, 20, 40]), ctx_len=32, pin=False)
    ids, labels = batch["input_ids"], batch["labels"]
    assert ids.shape == labels.shape == (3, 32) and ids.dtype == labels.dtype == torch.long      # 40 cut to ctx_len 32
    assert ids[0, :5].tolist() == [1, 2, 3, 4, 5] and ids[0, 5:].eq(0).all() and labels[0, 5:].eq(-100).all()
    assert ids[2].tolist() == list(range(201, 233)) and labels[2, -1] == 233
    short = collate_batch(_rows(2, [3, 17]), ctx_len=64, pin=False)
    assert short["input_ids"].shape == (2, 32)                                                   # 17 rounds up to 32, not to 64


def test_ranks_split_every_epoch_without_overlap_and_reshuffle():
    seen = [epoch_indices(10, 0, 7, True, r, 4) for r in range(4)]
    assert all(len(s) == 3 for s in seen)                                  # 10 padded to 12 by wrapping around
    flat = [i for s in seen for i in s]
    assert set(flat) == set(range(10)) and len(flat) == 12
    assert epoch_indices(10, 0, 7, True, 0, 1) != epoch_indices(10, 1, 7, True, 0, 1)            # a new order per epoch
    assert epoch_indices(10, 3, 7, True, 0, 1) == epoch_indices(10, 3, 7, True, 0, 1)            # but a fixed one per seed
    assert epoch_indices(6, 5, 7, False, 1, 2) == [1, 3, 5]


@pytest.mark.parametrize("prefetch", [0, 2])
def test_epoch_iteration_skip_and_batch_count(prefetch):
    loader = BatchLoader(_rows(9), micro_bsz=2, ctx_len=16, shuffle=False, prefetch=prefetch, pin=False)
    assert loader.batches_per_epoch() == 4 and not loader.is_iterable                             # the ninth row is dropped
    first = [b["input_ids"][:, 0].tolist() for b in loader.iter_epoch(0)]
    assert first == [[1, 101], [201, 301], [401, 501], [601, 701]]
    resumed = [b["input_ids"][:, 0].tolist() for b in loader.iter_epoch(0, skip_batches=3)]
    assert resumed == first[3:]
    two = [BatchLoader(_rows(8), 2, 16, rank=r, world=2, shuffle=False, prefetch=prefetch, pin=False) for r in range(2)]
    a = [b["input_ids"][:, 0].tolist() for b in two[0].iter_epoch(0)]
    b = [b["input_ids"][:, 0].tolist() for b in two[1].iter_epoch(0)]
    assert a == [[1, 201], [401, 601]] and b == [[101, 301], [501, 701]] and two[0].batches_per_epoch() == 2


def test_iterable_datasets_are_split_by_position_and_have_no_length():
    class Stream:
        def __iter__(self):
            return iter(_rows(10))

    loader = BatchLoader(Stream(), micro_bsz=2, ctx_len=16, rank=1, world=2, prefetch=0, pin=False)
    assert loader.is_iterable and loader.batches_per_epoch() is None
    got = [b["input_ids"][:, 0].tolist() for b in loader.iter_epoch(0)]
    assert got == [[101, 301], [501, 701]]                                  # odd positions; the fifth odd row has no partner
    assert [b["input_ids"][:, 0].tolist() for b in loader.iter_epoch(0, skip_batches=1)] == got[1:]


def test_errors_inside_the_prefetch_thread_reach_the_consumer_and_early_exit_is_clean():
    class Broken:
        def __len__(self):
            return 6

        def __getitem__(self, i):
            if i == 4:
                raise KeyError("row 4 is corrupt")
            return _rows(6)[i]

    loader = BatchLoader(Broken(), micro_bsz=2, ctx_len=16, shuffle=False, prefetch=2, pin=False)
    it = loader.iter_epoch(0)
    assert next(it)["input_ids"].shape == (2, 16) and next(it) is not None
    with pytest.raises(KeyError, match="row 4"):
        next(it)
    good = BatchLoader(_rows(64), micro_bsz=2, ctx_len=16, shuffle=False, prefetch=2, pin=False)
    for i, _ in enumerate(good.iter_epoch(0)):            # leaving the loop early stops the producer thread
        if i == 1:
            break
