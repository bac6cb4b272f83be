"""Work identity and the exactly-once ledger (Python face of ``csrc/runtime/work_ledger.cpp``).

``build_work_identity`` derives the stable identity of one unit of work; the ledger validates the
producer -> dispatch -> release -> commit protocol the controller runs, so committed work is neither
lost nor repeated across failures and resumes (reference: aspec/work_lifecycle.py:35-434).
"""
from __future__ import annotations

import ctypes as C
import hashlib
import json
from typing import Any, Mapping, Optional, Sequence

from aspec_b200 import _native


class WorkLifecycleError(RuntimeError):
    pass


def build_work_identity(*, split: str, epoch: int, source_id: str) -> dict:
    payload = json.dumps({"epoch": int(epoch), "source_id": str(source_id), "split": str(split)},
                         sort_keys=True, separators=(",", ":"))
    work_id = "sha256:" + hashlib.sha256(payload.encode()).hexdigest()
    return {"work_id": work_id, "execution_id": work_id + ":attempt:0", "work_kind": str(split)}


def require_work_identity(metadata: Optional[Mapping[str, Any]]):
    if not isinstance(metadata, Mapping):
        raise WorkLifecycleError("work metadata is missing")
    try:
        work_id, execution_id, kind = metadata["work_id"], metadata["execution_id"], metadata["work_kind"]
    except KeyError as exc:
        raise WorkLifecycleError(f"work metadata lacks {exc.args[0]}") from None
    if not all(isinstance(v, str) and v for v in (work_id, execution_id, kind)):
        raise WorkLifecycleError("work identity fields must be non-empty strings")
    if not execution_id.startswith(work_id + ":attempt:"):
        raise WorkLifecycleError("execution_id does not belong to work_id")
    return work_id, execution_id, kind


def _b(s) -> bytes:
    return str(s).encode()


class WorkLifecycleLedger:
    def __init__(self) -> None:
        lib = _native.runtime()
        lib.ab_ledger_create.restype = C.c_void_p
        lib.ab_ledger_last_error.restype = C.c_char_p
        lib.ab_ledger_status.restype = C.c_char_p
        lib.ab_ledger_state_of.restype = C.c_char_p
        lib.ab_ledger_resident_outputs.restype = C.c_longlong
        lib.ab_ledger_resident_bytes.restype = C.c_longlong
        self._lib = lib
        self._h = C.c_void_p(lib.ab_ledger_create())

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.ab_ledger_destroy(self._h)
            self._h = None

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise WorkLifecycleError(self._lib.ab_ledger_last_error(self._h).decode())

    def register_outputs(self, outputs: Sequence[Mapping[str, Any]]) -> list:
        rows = []
        for out in outputs:
            work_id, execution_id, kind = require_work_identity(out.get("metadata"))
            key = out.get("feature_key", out.get("mooncake_key"))
            rows.append((execution_id, work_id, kind, str(out["data_id"]), str(key), int(out["size_bytes"])))
        n = len(rows)
        arr = lambda i: (C.c_char_p * n)(*[_b(r[i]) for r in rows])
        sizes = (C.c_longlong * n)(*[r[5] for r in rows])
        self._check(self._lib.ab_ledger_register(self._h, n, arr(0), arr(1), arr(2), arr(3), arr(4), sizes))
        return [r[0] for r in rows]

    def register_output(self, *, data_id: str, metadata, size_bytes: int, feature_key: str = None,
                        mooncake_key: str = None) -> str:
        return self.register_outputs([{"data_id": data_id, "metadata": metadata, "size_bytes": size_bytes,
                                       "feature_key": feature_key if feature_key is not None else mooncake_key}])[0]

    def mark_dispatched(self, metadata, *, expected_consumers: int) -> None:
        _, execution_id, _ = require_work_identity(metadata)
        self._check(self._lib.ab_ledger_mark_dispatched(self._h, _b(execution_id), int(expected_consumers)))

    def release_output(self, *, execution_id: str, data_id: str, participant: str, outcome: str,
                       feature_key: str = None, mooncake_key: str = None) -> None:
        key = feature_key if feature_key is not None else mooncake_key
        self._check(self._lib.ab_ledger_release(self._h, _b(execution_id), _b(data_id), _b(key), _b(participant),
                                                _b(outcome)))

    def begin_discard(self, metadata) -> None:
        _, execution_id, _ = require_work_identity(metadata)
        self._check(self._lib.ab_ledger_begin_discard(self._h, _b(execution_id)))

    def confirm_discarded(self, metadata_items) -> None:
        for metadata in metadata_items:
            _, execution_id, _ = require_work_identity(metadata)
            self._check(self._lib.ab_ledger_confirm_discarded(self._h, _b(execution_id)))

    def commit_optimizer_step(self, *, optimizer_step: int, execution_ids: Sequence[str], expected_unique: int,
                              expected_occurrences: int = 1) -> None:
        self._check(self._lib.ab_ledger_commit(self._h, C.c_longlong(int(optimizer_step)),
                                               _b("\n".join(execution_ids)), int(expected_unique),
                                               int(expected_occurrences)))

    def discard_released_uncommitted(self) -> int:
        return int(self._lib.ab_ledger_discard(self._h, 0, b""))

    def discard_after_owner_fence(self, execution_ids: Sequence[str]) -> int:
        n = int(self._lib.ab_ledger_discard(self._h, 1, _b("\n".join(execution_ids))))
        if n < 0:
            raise WorkLifecycleError(self._lib.ab_ledger_last_error(self._h).decode())
        return n

    def discard_all_after_owner_fence(self) -> int:
        return int(self._lib.ab_ledger_discard(self._h, 2, b""))

    def state_of(self, execution_id: str) -> str:
        return self._lib.ab_ledger_state_of(self._h, _b(execution_id)).decode()

    @property
    def resident_outputs(self) -> int:
        return int(self._lib.ab_ledger_resident_outputs(self._h))

    @property
    def resident_bytes(self) -> int:
        return int(self._lib.ab_ledger_resident_bytes(self._h))

    def status(self) -> dict:
        return json.loads(self._lib.ab_ledger_status(self._h).decode())

    def committed_work_ids(self) -> list:
        return self.status()["committed_work_ids"]
