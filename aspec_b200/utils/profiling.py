"""Profiling windows: a torch-profiler trace and a CUDA memory snapshot over a chosen range of optimizer steps,
written under ``<run>/traces`` (reference: aspec/utils/profiling.py).  Nothing here changes GPU settings; timing
numbers are never taken while a window is open."""
from __future__ import annotations

import os
from typing import Optional

import torch


class StepProfiler:
    """``profile_start_step <= step < profile_end_step`` is traced; ``memory_snapshot_step`` dumps the allocator
    history once.  Call ``step(i)`` at the start of every optimizer step and ``close()`` at the end."""

    def __init__(self, trace_dir: str, start_step: Optional[int] = None, end_step: Optional[int] = None,
                 memory_snapshot_step: Optional[int] = None, rank: int = 0, with_stack: bool = False):
        self.trace_dir, self.rank = trace_dir, rank
        self.start, self.end, self.mem_step = start_step, end_step, memory_snapshot_step
        self.with_stack = with_stack
        self._prof = None
        self._recording_memory = False
        self.written = []

    @property
    def active(self) -> bool:
        return self._prof is not None

    def step(self, i: int) -> None:
        cuda = torch.cuda.is_available()
        if self.mem_step is not None and cuda:
            if i == self.mem_step - 1 and not self._recording_memory:
                torch.cuda.memory._record_memory_history(max_entries=200000)
                self._recording_memory = True
            elif i == self.mem_step + 1 and self._recording_memory:
                os.makedirs(self.trace_dir, exist_ok=True)
                path = os.path.join(self.trace_dir, f"memory-step{self.mem_step}-rank{self.rank}.pickle")
                torch.cuda.memory._dump_snapshot(path)
                torch.cuda.memory._record_memory_history(enabled=None)
                self._recording_memory = False
                self.written.append(path)
        if self.start is None or self.end is None:
            return
        if i == self.start and self._prof is None:
            acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if cuda else [])
            self._prof = torch.profiler.profile(activities=acts, record_shapes=False, with_stack=self.with_stack)
            self._prof.__enter__()
        elif i == self.end and self._prof is not None:
            self._finish()

    def _finish(self) -> None:
        self._prof.__exit__(None, None, None)
        os.makedirs(self.trace_dir, exist_ok=True)
        path = os.path.join(self.trace_dir, f"trace-steps{self.start}-{self.end}-rank{self.rank}.json")
        self._prof.export_chrome_trace(path)
        self.written.append(path)
        self._prof = None

    def close(self) -> None:
        if self._prof is not None:
            self._finish()
        if self._recording_memory:
            torch.cuda.memory._record_memory_history(enabled=None)
            self._recording_memory = False
