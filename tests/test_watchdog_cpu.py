"""Host-side failure detection: heartbeats, votes and the step guard, driven by a fake clock (no GPU, no sleeping)."""
import pytest

from rwkvtune_b200.engine.watchdog import DictStore, Heartbeat, RankFailure, StepAborted, StepGuard, vote


class FakeClock:
    def __init__(self):
        self.t = 1000.0

    def __call__(self):
        return self.t

    def advance(self, dt):
        self.t += dt


def test_missed_heartbeat_is_reported_before_the_next_step():
    store, clock = DictStore(), FakeClock()
    hbs = [Heartbeat(store, r, 3, timeout_s=5.0, clock=clock) for r in range(3)]
    for h in hbs:
        h.beat()
    assert hbs[0].failed_ranks() == []
    clock.advance(4.0)
    hbs[0].beat()
    hbs[1].beat()                       # rank 2 has stopped
    clock.advance(2.0)
    assert hbs[0].failed_ranks() == [2]
    with pytest.raises(RankFailure) as err:
        hbs[1].assert_alive()
    assert err.value.ranks == [2]
    hbs[2].beat()                       # it comes back
    hbs[0].assert_alive()


def test_rank_that_never_joined_counts_as_failed():
    store, clock = DictStore(), FakeClock()
    hb = Heartbeat(store, 0, 2, timeout_s=5.0, clock=clock)
    hb.beat()
    assert hb.failed_ranks() == [1]
    with pytest.raises(RankFailure):
        hb.assert_alive()


def test_vote_unanimous_dissent_and_late_voter():
    store, clock = DictStore(), FakeClock()
    sleeps = []

    def sleep(dt):
        sleeps.append(dt)
        clock.advance(dt)

    # everyone says yes (rank 1 voted first)
    store.set("vote/7/1", "1")
    assert vote(store, 0, 2, 7, True, timeout_s=1.0, clock=clock, sleep=sleep) is True
    # a dissenting rank
    store.set("vote/8/1", "0")
    assert vote(store, 0, 2, 8, True, timeout_s=1.0, clock=clock, sleep=sleep) is False
    # own dissent
    store.set("vote/9/1", "1")
    assert vote(store, 0, 2, 9, False, timeout_s=1.0, clock=clock, sleep=sleep) is False
    # a voter that arrives late but inside the deadline
    calls = {"n": 0}
    real_check = store.check

    def check(keys):
        calls["n"] += 1
        if calls["n"] == 5:
            store.set("vote/10/1", "1")
        return real_check(keys)

    store.check = check
    assert vote(store, 0, 2, 10, True, timeout_s=1.0, clock=clock, sleep=sleep) is True
    store.check = real_check
    # a voter that never arrives: failure after the deadline, not a hang
    t0 = clock()
    assert vote(store, 0, 2, 11, True, timeout_s=0.5, clock=clock, sleep=sleep) is False
    assert clock() - t0 >= 0.5


def test_step_guard_raises_on_dead_peer_and_on_failed_step():
    store, clock = DictStore(), FakeClock()
    guards = [StepGuard(store, r, 2, agree=None, timeout_s=5.0, interval_s=1.0, clock=clock) for r in range(2)]
    for g in guards:
        g.hb.beat()
    guards[0].before_step()
    # votes through the store: both clean
    store.set("vote/1/1", "1")
    guards[0].after_step(True)
    # the peer reports an expired device wait
    store.set("vote/2/1", "0")
    with pytest.raises(StepAborted):
        guards[0].after_step(True)
    # the peer goes quiet: seen on the host before the next launch
    clock.advance(10.0)
    guards[0].hb.beat()
    with pytest.raises(RankFailure):
        guards[0].before_step()


def test_step_guard_uses_the_agreement_callable():
    seen = []

    def agree(ok):
        seen.append(ok)
        return ok and len(seen) < 2

    g = StepGuard(DictStore(), 0, 2, agree=agree, clock=FakeClock())
    g.after_step(True)
    with pytest.raises(StepAborted):
        g.after_step(True)
    assert seen == [True, True]
