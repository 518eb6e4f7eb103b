"""Host-side failure detection: per-rank heartbeats in the rendezvous store and a step vote.

The reference has no failure detection at all (no heartbeat, no rank-failure handling).  Here every
rank publishes a monotonically increasing heartbeat to a key-value store (the torch.distributed
TCPStore in production, any object with ``set``/``get`` in tests).  A rank whose heartbeat is older
than ``timeout_s`` is reported as failed; survivors learn this on the host *before* their next
kernel launch or collective, so nothing is left waiting on the device.  ``vote`` lets all ranks
agree on whether a step's device-side status words were clean.  Nothing here touches a GPU, and
failures are injected in tests by simply not calling ``beat`` / by raising on a rank.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class DictStore:
    """In-process stand-in for a TCPStore (used by tests and single-process runs)."""

    def __init__(self) -> None:
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d[key]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int]):
        super().__init__(f"ranks {ranks} stopped sending heartbeats")
        self.ranks = ranks


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 30.0, interval_s: float = 1.0,
                 clock=time.time, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.timeout_s, self.interval_s, self.clock, self.prefix = timeout_s, interval_s, clock, prefix
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self.store.set(self._key(self.rank), repr(self.clock()))

    def start(self) -> None:
        self.beat()

        def loop():
            while not self._stop.wait(self.interval_s):
                self.beat()

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)

    def failed_ranks(self) -> List[int]:
        now = self.clock()
        bad = []
        for r in range(self.world):
            try:
                ok = self.store.check([self._key(r)]) if hasattr(self.store, "check") else True
                last = float(self.store.get(self._key(r)).decode()) if ok else None
            except Exception:
                last = None
            if last is None or now - last > self.timeout_s:
                bad.append(r)
        return bad

    def assert_alive(self) -> None:
        bad = [r for r in self.failed_ranks() if r != self.rank]
        if bad:
            raise RankFailure(bad)


def vote(store, rank: int, world_size: int, step: int, ok: bool, timeout_s: float = 10.0, clock=time.time,
         sleep=time.sleep) -> bool:
    """All ranks publish their verdict for ``step``; returns True only if every rank said ok.
    A rank that never votes counts as a failure after ``timeout_s``."""
    store.set(f"vote/{step}/{rank}", "1" if ok else "0")
    deadline = clock() + timeout_s
    keys = [f"vote/{step}/{r}" for r in range(world_size)]
    while clock() < deadline:
        if store.check(keys):
            return all(store.get(k) == b"1" for k in keys)
        sleep(0.01)
    return False


class StepAborted(RuntimeError):
    """Some rank reported a failed step (an expired device-side wait, an exception) and all ranks stop together."""


class StepGuard:
    """What a trainer runs around every optimiser step when there is more than one rank.

    * ``start()`` launches the heartbeat thread of this rank (store keys ``hb/<rank>``).
    * ``before_step()`` checks the peers' heartbeats (at most once per ``interval_s``) and raises
      :class:`RankFailure` *on the host, before the next kernel or collective is launched* when one has gone quiet.
    * ``after_step(ok)`` is called once the step's result has been read back: ``ok`` says whether this rank's
      device status words were clean; the ranks agree (a MIN-reduction over the host-side control group, falling back
      to a vote through the store) and every rank raises :class:`StepAborted` if any of them was not.

    ``store`` needs ``set`` / ``get`` / ``check`` (a ``torch.distributed.TCPStore`` or :class:`DictStore`);
    ``agree`` is a callable ``bool -> bool`` (``DistContext.all_agree``) or None to vote through the store.
    """

    def __init__(self, store, rank: int, world_size: int, agree=None, timeout_s: float = 60.0, interval_s: float = 1.0,
                 clock=time.time):
        self.rank, self.world = rank, world_size
        self.store, self.agree, self.clock = store, agree, clock
        self.hb = Heartbeat(store, rank, world_size, timeout_s, interval_s, clock)
        self.interval_s = interval_s
        self._last_check = None
        self._step = 0
        self.vote_timeout_s = timeout_s

    def start(self) -> None:
        self.hb.start()

    def stop(self) -> None:
        self.hb.stop()

    def before_step(self) -> None:
        now = self.clock()
        if self._last_check is not None and now - self._last_check < self.interval_s:
            return
        self._last_check = now
        self.hb.assert_alive()

    def after_step(self, ok: bool) -> None:
        self._step += 1
        if self.agree is not None:
            everyone = self.agree(bool(ok))
        else:
            everyone = vote(self.store, self.rank, self.world, self._step, bool(ok), self.vote_timeout_s, self.clock)
        if not everyone:
            raise StepAborted(f"rank {self.rank}: step {self._step} failed on "
                              f"{'this rank' if not ok else 'another rank'}; all ranks stop")
