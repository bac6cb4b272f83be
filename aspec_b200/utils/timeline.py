"""Per-process JSONL timeline of events and spans (``time.monotonic_ns``); a disabled recorder is a no-op
(reference: aspec/utils/timeline.py:76-286)."""
from __future__ import annotations

import json
import os
import threading
import time
from contextlib import contextmanager
from typing import Optional


class Timeline:
    def __init__(self, output_dir: Optional[str] = None, role: str = "driver", rank: int = 0, run_id: str = "",
                 flush_every: int = 128, enabled: bool = True):
        self.enabled = bool(enabled and output_dir)
        self.role, self.rank, self.run_id = role, rank, run_id
        self._buf, self._lock, self._flush_every = [], threading.Lock(), max(int(flush_every), 1)
        self._file = None
        if self.enabled:
            os.makedirs(output_dir, exist_ok=True)
            self._file = open(os.path.join(output_dir, f"timeline-{role}-{rank}-{os.getpid()}.jsonl"), "a")

    def event(self, name: str, **fields) -> None:
        if not self.enabled:
            return
        rec = {"t_ns": time.monotonic_ns(), "name": name, "role": self.role, "rank": self.rank, "pid": os.getpid(),
               "run_id": self.run_id, **fields}
        with self._lock:
            self._buf.append(json.dumps(rec, default=str))
            if len(self._buf) >= self._flush_every:
                self._flush_locked()

    @contextmanager
    def span(self, name: str, **fields):
        t0 = time.monotonic_ns()
        try:
            yield
        finally:
            self.event(name, duration_ns=time.monotonic_ns() - t0, **fields)

    def _flush_locked(self) -> None:
        if self._file and self._buf:
            self._file.write("\n".join(self._buf) + "\n")
            self._file.flush()
            self._buf.clear()

    def close(self) -> None:
        with self._lock:
            self._flush_locked()
            if self._file:
                self._file.close()
                self._file = None


def timeline_from_env(role: str, rank: int = 0) -> Timeline:
    """Settings travel to child processes through the environment (ASPEC_TIMELINE_DIR / _RUN_ID / _FLUSH)."""
    d = os.environ.get("ASPEC_TIMELINE_DIR")
    return Timeline(d, role, rank, os.environ.get("ASPEC_TIMELINE_RUN_ID", ""),
                    int(os.environ.get("ASPEC_TIMELINE_FLUSH", "128")), enabled=bool(d))
