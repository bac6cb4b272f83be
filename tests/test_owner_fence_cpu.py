"""Ownership fence: owners of shared memory are released only after every accessor process was observed dead."""
import multiprocessing as mp
import os
import time

import pytest

from aspec_b200.owner_fence import (ProcessIdentity, SourceFence, SourceFenceUnverified, observe_dead,
                                    run_with_source_fencing)


def _sleep_forever():
    while True:
        time.sleep(0.05)


class _Actor:
    """Just enough of a process actor: pid, shutdown, terminate."""

    def __init__(self, name, stubborn=False):
        self.name, self.stubborn = name, stubborn
        self.proc = mp.get_context("spawn").Process(target=_sleep_forever, daemon=True)
        self.proc.start()
        self.stopped_at = None

    @property
    def pid(self):
        return self.proc.pid

    def shutdown(self, timeout=1.0):
        self.terminate()

    def terminate(self):
        if self.stubborn:
            return                                        # a process the driver cannot bring down
        self.proc.terminate()
        self.proc.join(5)
        self.stopped_at = time.monotonic()

    def really_kill(self):
        self.proc.kill()
        self.proc.join(5)


def test_identity_tells_a_recycled_pid_from_the_original():
    me = ProcessIdentity.of(os.getpid(), "self")
    assert me.alive()
    assert not ProcessIdentity(os.getpid(), me.create_time - 100.0).alive()      # same pid, other start time
    assert not ProcessIdentity.of(2 ** 22 + 12345).alive()
    assert observe_dead([ProcessIdentity.of(2 ** 22 + 12345)], timeout=0.1) == []


def test_accessors_die_before_owners_are_released():
    engine, trainer = _Actor("engine"), _Actor("trainer")
    fence = SourceFence(grace_seconds=2.0, hold_seconds=2.0)
    fence.add_accessor(engine)
    fence.add_owner(trainer)
    fence.close(failed=True)
    assert fence.released and not engine.proc.is_alive() and not trainer.proc.is_alive()
    assert engine.stopped_at <= trainer.stopped_at


def test_unverifiable_accessor_keeps_the_owner_alive():
    engine, trainer = _Actor("engine", stubborn=True), _Actor("trainer")
    messages = []
    fence = SourceFence(grace_seconds=0.2, hold_seconds=0.5, log=messages.append)
    fence.add_accessor(engine)
    fence.add_owner(trainer)
    try:
        with pytest.raises(SourceFenceUnverified):
            fence.close(failed=True)
        assert not fence.released and trainer.proc.is_alive()          # memory owner untouched
        assert any("could not verify" in m for m in messages)
    finally:
        engine.really_kill()
        trainer.really_kill()


def test_run_with_source_fencing_closes_on_failure_and_chains_the_cause():
    made = {}

    def body(fence):
        made["engine"], made["trainer"] = _Actor("engine"), _Actor("trainer")
        fence.add_accessor(made["engine"])
        fence.add_owner(made["trainer"])
        raise ValueError("step failed")

    with pytest.raises(ValueError):
        run_with_source_fencing(body, fence=SourceFence(grace_seconds=2.0, hold_seconds=2.0))
    assert not made["engine"].proc.is_alive() and not made["trainer"].proc.is_alive()

    def stubborn_body(fence):
        made["engine"], made["trainer"] = _Actor("engine", stubborn=True), _Actor("trainer")
        fence.add_accessor(made["engine"])
        fence.add_owner(made["trainer"])
        raise ValueError("step failed")

    try:
        with pytest.raises(SourceFenceUnverified) as info:
            run_with_source_fencing(stubborn_body, fence=SourceFence(grace_seconds=0.2, hold_seconds=0.4))
        assert isinstance(info.value.__cause__, ValueError)
        assert made["trainer"].proc.is_alive()
    finally:
        made["engine"].really_kill()
        made["trainer"].really_kill()
