"""Ownership fence: memory that other processes can reach is released only after those processes are observed dead.

Feature rings live in the memory of the Draft trainer that consumes them and are written by Target engine
processes (GEMM epilogue stores over NVLink); slot tensors shared through queues are read by trainers.  When a
run fails, the owner of such memory must not free it while a process that can still touch it is alive: a late
store into freed device memory is a fault on somebody else's GPU.  So teardown is ordered - every *accessor* of
a region is asked to stop, then terminated, then **observed dead** (pid gone, or the pid now belongs to a
different process) - and only then is the *owner* allowed to exit.  If death cannot be verified within the hold
time the owners are kept alive and ``SourceFenceUnverified`` is raised for the operator.

The reference implements the same rule for Ray actors with a node-pinned psutil probe
(aspec/ray/owner_fence.py:42-151, entered from aspec/train_entry.py:523-526).  Here every role is a child
process of the driver on one node, so the probe is a direct psutil query.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Sequence

import psutil


class SourceFenceUnverified(RuntimeError):
    """Accessor processes could not be observed dead; the owners of the memory were left running."""


@dataclass(frozen=True)
class ProcessIdentity:
    """A pid together with its start time, so that a recycled pid is not mistaken for the original process."""
    pid: int
    create_time: float
    name: str = ""

    @classmethod
    def of(cls, pid: int, name: str = "") -> "ProcessIdentity":
        try:
            return cls(pid, psutil.Process(pid).create_time(), name)
        except (psutil.NoSuchProcess, psutil.AccessDenied):
            return cls(pid, -1.0, name)

    def alive(self) -> bool:
        if self.create_time < 0:
            return False
        try:
            p = psutil.Process(self.pid)
            return p.create_time() == self.create_time and p.status() != psutil.STATUS_ZOMBIE
        except psutil.NoSuchProcess:
            return False
        except psutil.AccessDenied:
            return True                                   # cannot tell: treat as alive


def observe_dead(identities: Iterable[ProcessIdentity], timeout: float, poll: float = 0.05) -> List[ProcessIdentity]:
    """Wait until every identity is dead; returns the ones still alive when ``timeout`` ran out."""
    pending = [i for i in identities if i.alive()]
    deadline = time.monotonic() + timeout
    while pending and time.monotonic() < deadline:
        time.sleep(poll)
        pending = [i for i in pending if i.alive()]
    return pending


class SourceFence:
    """Registry of who owns and who can reach shared memory, and the ordered teardown over it.

    ``add_accessor`` / ``add_owner`` take anything with ``pid`` (property or attribute), ``shutdown(timeout)`` and
    ``terminate()`` - a ``runtime.actor.ProcessActor`` - or a bare :class:`ProcessIdentity` (a process this driver
    did not start and cannot signal; it can only be waited for).
    """

    def __init__(self, *, grace_seconds: float = 5.0, hold_seconds: float = 60.0, log: Optional[Callable[[str], None]] = None):
        self.grace, self.hold = grace_seconds, hold_seconds
        self._accessors: list = []
        self._owners: list = []
        self._log = log or (lambda msg: None)
        self.released = False

    @staticmethod
    def _identity(actor) -> ProcessIdentity:
        if isinstance(actor, ProcessIdentity):
            return actor
        return ProcessIdentity.of(int(actor.pid), getattr(actor, "name", ""))

    def add_accessor(self, actor) -> None:
        self._accessors.append((actor, self._identity(actor)))

    def add_owner(self, actor) -> None:
        self._owners.append((actor, self._identity(actor)))

    def accessors(self) -> Sequence[ProcessIdentity]:
        return [i for _, i in self._accessors]

    def close(self, *, failed: bool = False) -> None:
        """Stop accessors, verify their death, then let the owners go.  ``failed`` skips the polite shutdown."""
        for actor, ident in self._accessors:
            if isinstance(actor, ProcessIdentity):
                continue
            try:
                if failed:
                    actor.terminate()
                else:
                    actor.shutdown(timeout=self.grace)
            except Exception as exc:                      # noqa: BLE001 - teardown continues, death is verified below
                self._log(f"fence: stopping {ident.name or ident.pid} raised {exc!r}")
        alive = observe_dead(self.accessors(), self.grace)
        for actor, ident in self._accessors:             # second attempt for the stragglers we can signal
            if ident in alive and not isinstance(actor, ProcessIdentity):
                try:
                    actor.terminate()
                except Exception:                         # noqa: BLE001
                    pass
        alive = observe_dead(alive, self.hold) if alive else []
        if alive:
            names = ", ".join(f"{i.name or 'pid'}:{i.pid}" for i in alive)
            self._log(f"fence: could not verify the death of {names}; owners stay alive")
            raise SourceFenceUnverified(f"accessors still alive after {self.hold}s: {names}; shared memory was not released")
        for actor, ident in self._owners:
            if isinstance(actor, ProcessIdentity):
                continue
            try:
                actor.shutdown(timeout=self.grace)
            except Exception as exc:                      # noqa: BLE001
                self._log(f"fence: stopping owner {ident.name or ident.pid} raised {exc!r}")
        self.released = True


def run_with_source_fencing(fn: Callable, *args, fence: Optional[SourceFence] = None, **kwargs):
    """Run ``fn(*args, fence=fence, **kwargs)``; whatever happens, close the fence before returning or re-raising.

    If the fence cannot be verified after a failure the original exception is chained to
    :class:`SourceFenceUnverified` and the driver process keeps the owners (its children) alive: the caller decides
    when to exit, and with it when the children's memory goes away.
    """
    fence = fence or SourceFence()
    try:
        result = fn(*args, fence=fence, **kwargs)
    except BaseException as exc:
        try:
            fence.close(failed=True)
        except SourceFenceUnverified as unverified:
            raise unverified from exc
        raise
    fence.close(failed=False)
    return result


def driver_identity() -> ProcessIdentity:
    return ProcessIdentity.of(os.getpid(), "driver")
