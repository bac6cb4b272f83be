"""Shared Target for several Drafts: one producer stream fans out to N experiments.

Every experiment runs its own training loop, controller (ledger, checkpoints) and trainer group, but all of them
plan the same rows in the same order (same dataset, seed, row shape).  The shared source merges the submissions
of one row from all live experiments into ONE Target pass whose epilogues store into every experiment's ring slot
(each reader may keep a subset of the captured layers), and hands every experiment its own view of the result.
Reader rights on all rings are acquired before the row is produced, so no consumer can see a key whose sibling
slot is not leased.  A failed or cancelled experiment is fenced: it leaves the live set, rows waiting only for it
are released to its siblings, and its submissions are ignored from then on
(reference: aspec/controller/shared_source.py:88-573, aspec/multi_draft.py:323-366).
"""
from __future__ import annotations

import copy
import threading
from typing import Callable, Dict, List, Sequence, Tuple

from aspec_b200.utils.types import InferenceOutput, RowRequest


class SharedSourceState:
    def __init__(self, manager, experiments: Sequence[str], consumer_offsets: Dict[str, int]):
        self.manager = manager
        self.live = list(experiments)
        self.offsets = dict(consumer_offsets)
        self._lock = threading.Lock()
        self._pending: Dict[str, Dict[str, Tuple[RowRequest, Tuple[int, ...]]]] = {}
        self._routes: Dict[str, List[Tuple[str, set]]] = {}             # row -> [(experiment, its global consumers)]
        self._callbacks: Dict[str, Callable] = {}
        self.rows_shared = 0
        self.fenced: Dict[str, str] = {}
        manager.on_result = self._on_result
        manager.on_consumer_stalled = self._stalled

    # -- experiment side ------------------------------------------------------------------------------
    def proxy(self, experiment: str) -> "ExperimentManager":
        return ExperimentManager(self, experiment)

    def submit(self, experiment: str, request: RowRequest, consumers: Sequence[int]) -> None:
        with self._lock:
            if experiment not in self.live:
                return
            entry = self._pending.setdefault(request.row_id, {})
            if entry:
                first = next(iter(entry.values()))[0]
                if list(first.data_ids) != list(request.data_ids):
                    raise RuntimeError(f"experiments disagree on the content of {request.row_id}: "
                                       f"{first.data_ids} vs {request.data_ids}")
            entry[experiment] = (request, tuple(consumers))
            self._flush_ready()

    def _stalled(self, consumer: int, seconds: float) -> bool:
        """A reader freed no ring slot for ``seconds``: its experiment leaves the stream, the others go on."""
        owner = max((n for n in self.offsets if self.offsets[n] <= consumer), key=lambda n: self.offsets[n], default=None)
        if owner is None or owner not in self.live or len(self.live) < 2:
            return False                      # the last reader standing: the stream has nobody else to serve
        self.fence(owner, f"stalled: consumer {consumer} freed no ring slot within {seconds:.0f} s")
        return True

    def fence(self, experiment: str, reason: str) -> None:
        """Remove an experiment; rows that only waited for it go to its siblings."""
        with self._lock:
            if experiment in self.live:
                self.live.remove(experiment)
                self.fenced[experiment] = reason
                # its consumers are [its offset, the next experiment's offset)
                end = min([c for c in self.offsets.values() if c > self.offsets[experiment]] + [10 ** 9])
                self.manager.dead_consumers |= {c for c in self.manager.rings
                                                if self.offsets[experiment] <= c < end}
                for entry in self._pending.values():
                    entry.pop(experiment, None)
                self._flush_ready()

    def _flush_ready(self) -> None:
        for row_id in [r for r, e in self._pending.items() if e and all(x in e for x in self.live)]:
            entry = self._pending.pop(row_id)
            names = [x for x in self.live if x in entry]
            if not names:
                continue
            base = entry[names[0]][0]
            merged = copy.copy(base)
            merged.layer_ids = tuple(sorted({l for n in names for l in entry[n][0].layer_ids}))
            consumers, routes = [], []
            for n in names:
                mine = [self.offsets[n] + c for c in entry[n][1]]
                routes.append((n, set(mine)))
                consumers += mine
            self._routes[row_id] = routes
            self.rows_shared += 1
            self.manager.submit(merged, consumers)

    # -- producer side --------------------------------------------------------------------------------
    def _on_result(self, out: InferenceOutput, req: RowRequest) -> None:
        with self._lock:
            routes = self._routes.pop(out.row_id, [])
            callbacks = dict(self._callbacks)
            live = set(self.live)
        for name, mine in routes:
            if name not in live or name not in callbacks:
                continue                     # fenced after submission: its leases die with its rings
            picks = [i for i, (c, _s, _g) in enumerate(req.leases) if c in mine]
            if len(picks) != len(mine):
                continue
            view_out, view_req = copy.copy(out), copy.copy(req)
            view_out.feature_keys = [out.feature_keys[i] for i in picks]
            view_req.leases = [(req.leases[i][0] - self.offsets[name], req.leases[i][1], req.leases[i][2]) for i in picks]
            callbacks[name](view_out, view_req)

    def status(self) -> dict:
        return {"live": list(self.live), "fenced": dict(self.fenced), "rows_shared": self.rows_shared,
                "pending_rows": len(self._pending)}


class ExperimentManager:
    """What one experiment's training loop sees in place of the inference manager."""

    def __init__(self, state: SharedSourceState, experiment: str):
        self._state, self.experiment = state, experiment

    @property
    def on_result(self):
        return self._state._callbacks.get(self.experiment)

    @on_result.setter
    def on_result(self, fn) -> None:
        self._state._callbacks[self.experiment] = fn

    def submit(self, request: RowRequest, consumers: Sequence[int]) -> None:
        self._state.submit(self.experiment, request, consumers)

    def raise_if_failed(self) -> None:
        self._state.manager.raise_if_failed()
        if self.experiment in self._state.fenced:
            raise RuntimeError(f"experiment {self.experiment} was fenced: {self._state.fenced[self.experiment]}")

    def idle(self) -> bool:
        return self._state.manager.idle()

    def error(self):
        return self._state.manager.error()
