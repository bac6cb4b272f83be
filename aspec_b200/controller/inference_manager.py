"""Producer side of the pipeline: leases ring slots, drives the engines, forwards descriptors in order.

Role of the reference's ``AsyncInferenceManager`` (aspec/controller/inference_manager.py:341-1324).  A
background thread takes planned rows in plan order, acquires a destination lease per consumer (the
bounded rings are the back-pressure: ``acquire`` blocks while a consumer still owns all its slots), sends
batches of rows to the least-loaded engine, and hands every finished row to ``on_result`` - strictly in
submission order, so a trainer's queue always holds the rows of micro-step ``m`` before those of ``m+1``.
An engine failure is latched and re-raised in the training loop.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

from aspec_b200.runtime.actor import ProcessActor
from aspec_b200.transport.slot_ring import GenerationSlotRing
from aspec_b200.utils.types import InferenceOutput, RowRequest


class InferenceManager:
    def __init__(self, engines: Sequence, rings: Dict[int, GenerationSlotRing], on_result: Callable[[InferenceOutput, RowRequest], None],
                 batch_size: int = 1, acquire_timeout: float = 120.0, max_inflight_per_engine: int = 2,
                 batch_tokens: int = 0):
        self.engines = list(engines)
        self.rings = rings
        self.on_result = on_result
        self.batch_size = max(int(batch_size), 1)
        # > 0: a batch is sent once it holds this many tokens (or ``batch_size`` rows, whichever comes first), so that
        # batches of short documents still give the Target full-width GEMMs
        self.batch_tokens = max(int(batch_tokens), 0)
        self.acquire_timeout = acquire_timeout
        self.max_inflight = max_inflight_per_engine
        self._todo: "queue.Queue" = queue.Queue()
        self._error: Optional[BaseException] = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="inference-manager", daemon=True)
        self._inflight: List[tuple] = []          # (future, requests) in submission order
        self.submitted = 0
        self.completed = 0
        self._engine_load = [0] * len(self.engines)
        self.dead_consumers: set = set()          # fenced readers: never leased again, pending waits are abandoned
        # ``f(consumer, seconds) -> bool``: called when a consumer freed no slot in time; True = it was fenced, go on
        self.on_consumer_stalled: Optional[Callable[[int, float], bool]] = None

    def start(self) -> None:
        self._thread.start()

    def submit(self, request: RowRequest, consumers: Sequence[int]) -> None:
        """Queue one row for the given consumer ranks (several = shared-Target fan-out)."""
        self._todo.put((request, tuple(consumers)))
        self.submitted += 1

    def error(self) -> Optional[BaseException]:
        return self._error

    def raise_if_failed(self) -> None:
        if self._error is not None:
            raise RuntimeError(f"inference manager failed: {self._error}") from self._error

    def idle(self) -> bool:
        return self._todo.empty() and not self._inflight

    def stop(self) -> None:
        self._stop.set()
        self._todo.put(None)
        self._thread.join(timeout=10.0)

    # -- worker -------------------------------------------------------------------------------------
    def _call(self, engine, method, *args):
        if isinstance(engine, ProcessActor):
            return engine.call_async(method, *args)
        result = getattr(engine, method)(*args)

        class _Done:
            def get(self, timeout=None):
                return result

            def done(self):
                return True
        return _Done()

    def _pick_engine(self) -> int:
        """Least-loaded engine; among equally loaded ones the one after the last pick, so that a stream of rows that
        arrive one at a time (long-context runs) rotates over all Target GPUs instead of always taking the first."""
        n = len(self.engines)
        start = (getattr(self, "_last_engine", -1) + 1) % n
        order = [(start + i) % n for i in range(n)]
        eng = min(order, key=lambda i: self._engine_load[i])
        self._last_engine = eng
        return eng

    def _collect(self, block: bool) -> None:
        while self._inflight:
            fut, reqs, eng = self._inflight[0]
            if not block and not fut.done():
                return
            outs = fut.get(timeout=self.acquire_timeout * 4)
            self._inflight.pop(0)
            self._engine_load[eng] -= 1
            for out, req in zip(outs, reqs):
                self.on_result(out, req)
                self.completed += 1
            block = False

    def _run(self) -> None:
        batch: List[RowRequest] = []

        def flush() -> None:
            nonlocal batch
            if not batch:
                return
            eng = self._pick_engine()
            while self._engine_load[eng] >= self.max_inflight:
                self._collect(block=True)
                eng = self._pick_engine()
            self._inflight.append((self._call(self.engines[eng], "generate", batch), batch, eng))
            self._engine_load[eng] += 1
            batch = []

        try:
            while not self._stop.is_set():
                try:
                    item = self._todo.get(timeout=0.02)
                except queue.Empty:
                    item = "idle"
                if item is None:
                    break
                if item != "idle":
                    request, consumers = item
                    leases = []
                    for c in consumers:
                        deadline = time.monotonic() + self.acquire_timeout
                        while True:
                            if c in self.dead_consumers:
                                lease = None
                                break
                            try:
                                lease = self.rings[c].acquire(f"row:{request.row_id}", timeout=0.05)
                                break
                            except TimeoutError:
                                # the consumer still owns all its slots: get the rows already leased to the
                                # engines (the consumer may be waiting for exactly those) and keep collecting
                                flush()
                                self._collect(block=False)
                                if time.monotonic() > deadline or self._stop.is_set():
                                    # several independent readers share this stream: one that stopped consuming is
                                    # taken out (its owner decides) instead of ending the stream for all of them
                                    if self.on_consumer_stalled is not None and not self._stop.is_set() \
                                            and self.on_consumer_stalled(c, self.acquire_timeout) and c in self.dead_consumers:
                                        lease = None
                                        break
                                    raise TimeoutError(
                                        f"no free ring slot on consumer {c} within {self.acquire_timeout}s") from None
                        if lease is not None:
                            leases.append((c, lease.slot_id, lease.generation))
                    request.leases = leases
                    if leases:
                        batch.append(request)
                full = len(batch) >= self.batch_size or (self.batch_tokens > 0 and batch
                                                         and sum(sum(r.document_lengths) for r in batch) >= self.batch_tokens)
                if full or item == "idle":
                    flush()
                self._collect(block=False)
            if not self._stop.is_set():
                flush()
                self._collect(block=True)
        except BaseException as exc:                 # noqa: BLE001 - latched for the training loop
            self._error = exc
