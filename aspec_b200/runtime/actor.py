"""Process actors: one OS process per GPU role, driven by method calls from the driver.

The reference orchestrates Ray actors (aspec/ray/ray_actor.py:56-106, aspec/ray/train_group.py:76-365).
On one B200 node every role is a child process of the driver, so an actor here is a
``torch.multiprocessing`` process that serves ``(method, args, kwargs)`` requests from a pipe; tensors
that travel through queues are shared (CUDA IPC or shared memory), never copied through the pipe.
A call has a deadline; an actor that raised reports the traceback; ``terminate`` kills the process
(the fence the driver applies before it reclaims memory the actor might still touch).
"""
from __future__ import annotations

import os
import threading
import time
import traceback
from typing import Any, Callable, Dict, List, Optional

import torch.multiprocessing as mp

_CTX = mp.get_context("spawn")


class ActorError(RuntimeError):
    pass


class ActorTimeout(TimeoutError):
    pass


def _serve(factory, factory_args, factory_kwargs, conn, env: Dict[str, str]) -> None:
    os.environ.update(env)
    try:
        obj = factory(*factory_args, **factory_kwargs)
        conn.send(("ready", None))
    except BaseException:                                           # noqa: BLE001 - reported to the driver
        conn.send(("error", traceback.format_exc()))
        return
    while True:
        try:
            msg = conn.recv()
        except (EOFError, KeyboardInterrupt):
            break
        if msg is None:
            break
        call_id, method, args, kwargs = msg
        try:
            result = getattr(obj, method)(*args, **kwargs)
            conn.send((call_id, "ok", result))
        except BaseException:                                       # noqa: BLE001
            conn.send((call_id, "error", traceback.format_exc()))
    close = getattr(obj, "close", None)
    if callable(close):
        try:
            close()
        except Exception:                                           # noqa: BLE001
            pass


class Future:
    def __init__(self, actor: "ProcessActor", call_id: int, method: str):
        self.actor, self.call_id, self.method = actor, call_id, method

    def get(self, timeout: Optional[float] = None) -> Any:
        return self.actor._wait(self.call_id, self.method, timeout)

    def done(self) -> bool:
        return self.actor._poll(self.call_id)


class ProcessActor:
    """``ProcessActor(factory, *args, env={...})`` starts the process and constructs ``factory(*args)`` in it."""

    def __init__(self, factory: Callable, *args, name: str = "actor", env: Optional[Dict[str, str]] = None,
                 start_timeout: float = 600.0, **kwargs):
        self.name = name
        self._parent, child = _CTX.Pipe()
        self._proc = _CTX.Process(target=_serve, args=(factory, args, kwargs, child, dict(env or {})),
                                  name=name, daemon=True)
        self._proc.start()
        self._lock = threading.Lock()
        self._next = 0
        self._results: Dict[int, tuple] = {}
        self._start_timeout = start_timeout
        self._ready = False

    def wait_ready(self) -> "ProcessActor":
        if self._ready:
            return self
        if not self._parent.poll(self._start_timeout):
            raise ActorTimeout(f"{self.name} did not start within {self._start_timeout}s")
        try:
            kind, payload = self._parent.recv()
        except (EOFError, OSError):
            self._proc.join(1.0)
            raise ActorError(f"{self.name} exited (code {self._proc.exitcode}) before it was ready "
                             "(a negative code is the signal that killed it, e.g. -9 when the host ran out of memory)") from None
        if kind != "ready":
            raise ActorError(f"{self.name} failed to start:\n{payload}")
        self._ready = True
        return self

    @property
    def pid(self) -> int:
        return self._proc.pid

    def is_alive(self) -> bool:
        return self._proc.is_alive()

    def call_async(self, method: str, *args, **kwargs) -> Future:
        self.wait_ready()
        with self._lock:
            call_id = self._next
            self._next += 1
            self._parent.send((call_id, method, args, kwargs))
        return Future(self, call_id, method)

    def call(self, method: str, *args, timeout: Optional[float] = None, **kwargs) -> Any:
        return self.call_async(method, *args, **kwargs).get(timeout)

    def _drain(self, block_for: Optional[float]) -> None:
        if self._parent.poll(block_for):
            call_id, status, payload = self._parent.recv()
            self._results[call_id] = (status, payload)

    def _poll(self, call_id: int) -> bool:
        with self._lock:
            try:
                while self._parent.poll(0):
                    self._drain(0)
            except (EOFError, OSError):
                return True               # the process is gone: ``get`` reports how it ended
            return call_id in self._results

    def _wait(self, call_id: int, method: str, timeout: Optional[float]) -> Any:
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            with self._lock:
                if call_id in self._results:
                    status, payload = self._results.pop(call_id)
                    if status == "error":
                        raise ActorError(f"{self.name}.{method} raised:\n{payload}")
                    return payload
                remaining = 0.05 if deadline is None else min(0.05, max(deadline - time.monotonic(), 0.0))
                try:
                    self._drain(remaining)
                except (EOFError, OSError):
                    self._proc.join(1.0)
                    raise ActorError(f"{self.name} exited (code {self._proc.exitcode}) during {method}") from None
            if not self._proc.is_alive() and not self._parent.poll(0):
                raise ActorError(f"{self.name} exited (code {self._proc.exitcode}) during {method}")
            if deadline is not None and time.monotonic() >= deadline:
                raise ActorTimeout(f"{self.name}.{method} exceeded {timeout}s")

    def shutdown(self, timeout: float = 10.0) -> None:
        if self._proc.is_alive():
            try:
                self._parent.send(None)
            except (OSError, BrokenPipeError):
                pass
            self._proc.join(timeout)
        self.terminate()

    def terminate(self) -> None:
        """Kill the process.  After this returns the process can no longer touch shared memory."""
        if self._proc.is_alive():
            self._proc.terminate()
            self._proc.join(5.0)
            if self._proc.is_alive():
                self._proc.kill()
                self._proc.join(5.0)


class _JoinedFuture:
    """Done when every member's call is done; the result is the first member's."""

    def __init__(self, futures: List[Future]):
        self.futures = futures

    def done(self) -> bool:
        return all(f.done() for f in self.futures)

    def get(self, timeout: Optional[float] = None) -> Any:
        # a member that died leaves its peers waiting for it inside a collective: its exit is reported at once instead
        # of after their timeout
        deadline = None if timeout is None else time.monotonic() + timeout
        results: Dict[int, Any] = {}
        while len(results) < len(self.futures):
            for i, f in enumerate(self.futures):
                if i not in results and f.done():
                    results[i] = f.get(1.0)
            if len(results) == len(self.futures):
                break
            for i, f in enumerate(self.futures):
                if i not in results and not f.actor.is_alive() and not f.done():
                    raise ActorError(f"{f.actor.name} exited (code {f.actor._proc.exitcode}) during {f.method}; "
                                     "the other members of its group cannot finish the call")
            if deadline is not None and time.monotonic() >= deadline:
                raise ActorTimeout(f"{self.futures[0].actor.name}.{self.futures[0].method} exceeded {timeout}s")
            time.sleep(0.005)
        return results[0]


class ActorGroup(ProcessActor):
    """Several actor processes that act as one: every call goes to all members (ranks of one tensor-parallel engine must
    all run every pass), completes when all have completed, and returns the first member's answer.  Stands wherever one
    ``ProcessActor`` does."""

    def __init__(self, members: List[ProcessActor], name: str = "group"):
        self.members = list(members)
        self.name = name

    def wait_ready(self) -> "ActorGroup":
        for m in self.members:
            m.wait_ready()
        return self

    @property
    def pid(self) -> int:
        return self.members[0].pid

    def is_alive(self) -> bool:
        return all(m.is_alive() for m in self.members)

    def call_async(self, method: str, *args, **kwargs) -> _JoinedFuture:
        return _JoinedFuture([m.call_async(method, *args, **kwargs) for m in self.members])

    def call(self, method: str, *args, timeout: Optional[float] = None, **kwargs) -> Any:
        return self.call_async(method, *args, **kwargs).get(timeout)

    def shutdown(self, timeout: float = 10.0) -> None:
        for m in self.members:
            m.shutdown(timeout)

    def terminate(self) -> None:
        for m in self.members:
            m.terminate()


def make_queue():
    return _CTX.Queue()


def wait_all(futures: List[Future], timeout: Optional[float] = None) -> List[Any]:
    deadline = None if timeout is None else time.monotonic() + timeout
    out = []
    for f in futures:
        out.append(f.get(None if deadline is None else max(deadline - time.monotonic(), 0.0)))
    return out
