"""Cooperative termination: SIGTERM / SIGINT become a ``TerminationRequested`` exception raised at a safe point,
and critical sections (checkpoint commit, ledger updates) can defer delivery until they finish
(reference: aspec/runtime_control.py:22-81)."""
from __future__ import annotations

import contextlib
import signal
import threading


class TerminationRequested(BaseException):
    def __init__(self, signum: int):
        super().__init__(f"termination requested by signal {signum}")
        self.signum = signum


_state = threading.local()
_pending = {"signum": None}
_depth = {"n": 0}


def _handler(signum, _frame):
    if _depth["n"] > 0:
        _pending["signum"] = signum
        return
    raise TerminationRequested(signum)


def install_termination_handlers(signals=(signal.SIGTERM, signal.SIGINT)) -> dict:
    """Install on the main thread; returns the previous handlers so a caller can restore them."""
    return {s: signal.signal(s, _handler) for s in signals}


def restore_handlers(previous: dict) -> None:
    for s, h in previous.items():
        signal.signal(s, h)


@contextlib.contextmanager
def deferred_termination():
    """Signals arriving inside the block are remembered and raised when the outermost block exits."""
    _depth["n"] += 1
    try:
        yield
    finally:
        _depth["n"] -= 1
        if _depth["n"] == 0 and _pending["signum"] is not None:
            signum, _pending["signum"] = _pending["signum"], None
            raise TerminationRequested(signum)


def termination_pending() -> bool:
    return _pending["signum"] is not None
