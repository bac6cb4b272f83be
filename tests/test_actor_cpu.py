"""Process actors and actor groups: calls, errors with the child's traceback, exits reported with their code, and a
group whose member dies fails the call at once instead of waiting on the survivors (reference: the Ray actor base,
aspec/ray/ray_actor.py:56-106, whose failures surface as RayActorError)."""
import os
import time

import pytest

from aspec_b200.runtime.actor import ActorError, ActorGroup, ActorTimeout, ProcessActor


class Worker:
    def __init__(self, rank: int):
        self.rank = rank

    def work(self, x):
        return (self.rank, x * 2)

    def slow(self, seconds):
        time.sleep(seconds)
        return self.rank

    def boom(self):
        raise ValueError(f"rank {self.rank} failed")

    def leave(self):
        os._exit(7)


@pytest.mark.timeout(120)
def test_calls_errors_timeouts_and_exits_of_one_actor():
    a = ProcessActor(Worker, 3, name="w3")
    try:
        assert a.call("work", 21, timeout=30) == (3, 42)
        with pytest.raises(ActorError, match="rank 3 failed"):
            a.call("boom", timeout=30)
        with pytest.raises(ActorTimeout):
            a.call("slow", 5.0, timeout=0.2)
        with pytest.raises(ActorError, match=r"exited \(code 7\)"):
            a.call("leave", timeout=30)
        assert not a.is_alive()
    finally:
        a.terminate()


@pytest.mark.timeout(120)
def test_a_group_answers_with_its_first_member_and_reports_a_dead_member_at_once():
    group = ActorGroup([ProcessActor(Worker, r, name=f"tp.{r}") for r in range(3)], name="tp")
    try:
        group.wait_ready()
        assert group.call("work", 5, timeout=30) == (0, 10) and group.is_alive() and group.pid == group.members[0].pid
        fut = group.call_async("slow", 0.3)
        assert not fut.done()
        assert fut.get(timeout=30) == 0
        # member 1 leaves while the others are still busy (as ranks stuck in a collective with it would be)
        busy = [group.members[0].call_async("slow", 20.0), group.members[2].call_async("slow", 20.0)]
        t0 = time.monotonic()
        from aspec_b200.runtime.actor import _JoinedFuture
        joined = _JoinedFuture([busy[0], group.members[1].call_async("leave"), busy[1]])
        with pytest.raises(ActorError, match=r"tp\.1 exited \(code 7\)"):
            joined.get(timeout=60)
        assert time.monotonic() - t0 < 10 and not group.is_alive()
    finally:
        group.terminate()
    assert not any(m.is_alive() for m in group.members)
