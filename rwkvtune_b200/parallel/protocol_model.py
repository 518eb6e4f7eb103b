"""Host-side model of the device flag protocols, for exhaustive interleaving checks.

The fused ZeRO-2 step (``rwkvtune_b200/csrc/zero_p2p.cu`` driven by :mod:`rwkvtune_b200.parallel.p2p`) orders
kernels of different GPUs with flag words: per-bucket "gradients complete" flags, and an epoch barrier.  A GPU
data race there would be silent (a reduce reading a peer's gradient bucket before it is complete, or after the
peer has cleared it for the next micro-batch).  The reference has nothing to check here: DeepSpeed/NCCL own its
ordering.  This module restates the protocol as per-rank, per-stream lists of abstract operations and explores
**every** interleaving of them (streams of one rank are sequential, streams of different ranks and the two
streams of one rank run concurrently, a wait blocks until its condition holds, an event orders two streams of a
rank), asserting at every read that the data it sees is the version the algorithm requires.  It runs on the CPU in
milliseconds for 2-3 ranks and 2-3 buckets and is the "model check of the flag protocols" of the test suite.

Operations (tuples):

``("write", bucket, version)``   gradient bucket of this rank now holds ``version`` (a micro-batch number)
``("signal", word, value)``      store ``value`` into ``flags[peer][word][rank]`` of every peer (release)
``("wait", word, value)``        block until ``flags[rank][word][p] >= value`` for every ``p`` (acquire)
``("read", bucket, version)``    owner reads the bucket of every rank; each must hold exactly ``version``
``("record", event)`` / ``("wait_event", event)``   stream ordering inside one rank
``("clear", bucket)``            the rank clears its bucket (version becomes -1)
"""
from __future__ import annotations

from typing import Dict, List, Tuple

Op = Tuple


class ProtocolViolation(AssertionError):
    pass


def explore(programs: List[Dict[str, List[Op]]], n_words: int, max_states: int = 2_000_000) -> int:
    """``programs[rank][stream]`` is a list of operations.  Explores all interleavings (depth-first, memoised on
    the full state) and returns the number of distinct states visited.  Raises :class:`ProtocolViolation` when a
    read sees a wrong version, and on deadlock (some stream blocked forever)."""
    W = len(programs)
    streams = [(r, s) for r in range(W) for s in programs[r]]
    n_buckets = 1 + max([op[1] for r in range(W) for s in programs[r] for op in programs[r][s]
                         if op[0] in ("write", "read", "clear")], default=0)

    def initial():
        pcs = tuple(0 for _ in streams)
        flags = tuple(tuple(tuple(0 for _ in range(W)) for _ in range(n_words)) for _ in range(W))
        data = tuple(tuple(-1 for _ in range(n_buckets)) for _ in range(W))
        events = tuple(frozenset() for _ in range(W))
        return pcs, flags, data, events

    seen = set()
    stack = [initial()]
    while stack:
        state = stack.pop()
        if state in seen:
            continue
        seen.add(state)
        if len(seen) > max_states:
            raise RuntimeError("state space larger than max_states")
        pcs, flags, data, events = state
        progressed, all_done = False, True
        for i, (r, s) in enumerate(streams):
            prog = programs[r][s]
            if pcs[i] >= len(prog):
                continue
            all_done = False
            op = prog[pcs[i]]
            kind = op[0]
            nflags, ndata, nevents = flags, data, events
            if kind == "wait":
                if not all(flags[r][op[1]][p] >= op[2] for p in range(W)):
                    continue
            elif kind == "wait_event":
                if op[1] not in events[r]:
                    continue
            elif kind == "signal":
                nflags = tuple(tuple(tuple(op[2] if (w == op[1] and q == r) else flags[p][w][q] for q in range(W))
                                     for w in range(n_words)) for p in range(W))
            elif kind == "write":
                ndata = tuple(tuple(op[2] if (p == r and b == op[1]) else data[p][b] for b in range(n_buckets))
                              for p in range(W))
            elif kind == "clear":
                ndata = tuple(tuple(-1 if (p == r and b == op[1]) else data[p][b] for b in range(n_buckets))
                              for p in range(W))
            elif kind == "read":
                got = [data[p][op[1]] for p in range(W)]
                if any(g != op[2] for g in got):
                    raise ProtocolViolation(f"rank {r} stream {s}: read of bucket {op[1]} expected version {op[2]} "
                                            f"from every rank, saw {got}")
            elif kind == "record":
                nevents = tuple(events[p] | {op[1]} if p == r else events[p] for p in range(W))
            else:
                raise ValueError(f"unknown operation {op!r}")
            npcs = tuple(pc + 1 if j == i else pc for j, pc in enumerate(pcs))
            stack.append((npcs, nflags, ndata, nevents))
            progressed = True
        if not progressed and not all_done:
            blocked = [(r, s, programs[r][s][pcs[i]]) for i, (r, s) in enumerate(streams) if pcs[i] < len(programs[r][s])]
            raise ProtocolViolation(f"deadlock: {blocked}")
    return len(seen)


def zero2_step_programs(world: int, n_buckets: int, owner_of_bucket, micro_batches: int = 2,
                        signal_before_write: bool = False, skip_micro_barrier: bool = False):
    """The fused ZeRO-2 protocol as operation lists: per micro-batch, every rank writes its buckets in reverse order
    (backward), signals each bucket, and the owner's side stream waits for all ranks' flags of that bucket and reads
    it; after a non-final micro-batch the ranks meet at the epoch barrier and clear their buckets; after the final one
    they meet at the barrier before anyone overwrites gradients again.  Flag words: ``0`` = barrier, ``1 + b`` =
    bucket ``b``.  ``signal_before_write`` and ``skip_micro_barrier`` build deliberately broken variants."""
    programs = []
    for r in range(world):
        compute, comm = [], []
        barrier_epoch = 0
        for m in range(micro_batches):
            epoch = m + 1
            for b in reversed(range(n_buckets)):
                ops = [("write", b, m), ("signal", 1 + b, epoch)]
                compute += ops[::-1] if signal_before_write else ops
                if owner_of_bucket(b) == r:
                    ev = f"b{b}e{epoch}"
                    compute.append(("record", ev))
                    comm += [("wait_event", ev), ("wait", 1 + b, epoch), ("read", b, m)]
            done = f"join{epoch}"
            comm.append(("record", done))
            compute.append(("wait_event", done))
            last = m == micro_batches - 1
            if not (skip_micro_barrier and not last):
                barrier_epoch += 1
                compute += [("signal", 0, barrier_epoch), ("wait", 0, barrier_epoch)]
            compute += [("clear", b) for b in range(n_buckets)]
        programs.append({"compute": compute, "comm": comm})
    return programs, 1 + n_buckets
