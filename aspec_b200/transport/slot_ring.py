"""Generation-checked slot ring (Python face of ``csrc/runtime/slot_ring.cpp``).

Protocol of the reference's ``GenerationSlotRing`` (aspec/transfer/mooncake/p2p.py:315-465): bounded
slots, leases ``(slot, generation, owner)``, a reader audience frozen before publication, idempotent
acknowledged release.  The generation is also what a consumer kernel waits for in the slot's device flag.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Iterable, Optional

from aspec_b200 import _native

_OK, _TIMEOUT, _STALE, _PENDING, _ALREADY_REG, _NOT_READER, _BAD, _ALREADY_ACK = range(8)


@dataclass(frozen=True)
class RingLease:
    slot_id: int
    generation: int
    owner: str


class GenerationSlotRing:
    def __init__(self, slots: int):
        if slots < 1:
            raise ValueError("slots must be at least 1")
        lib = _native.runtime()
        lib.ab_ring_create.restype = C.c_void_p
        self._lib = lib
        self._h = C.c_void_p(lib.ab_ring_create(int(slots)))
        self._slots = int(slots)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.ab_ring_destroy(self._h)
            self._h = None

    @property
    def slots(self) -> int:
        return self._slots

    @property
    def in_use(self) -> int:
        return int(self._lib.ab_ring_in_use(self._h))

    def wait_until_empty(self, timeout: Optional[float] = None) -> bool:
        return bool(self._lib.ab_ring_wait_until_empty(self._h, C.c_double(-1.0 if timeout is None else timeout)))

    def acquire(self, owner: str, timeout: Optional[float] = None) -> RingLease:
        slot, gen = C.c_int(), C.c_longlong()
        rc = self._lib.ab_ring_acquire(self._h, owner.encode(), C.c_double(-1.0 if timeout is None else timeout),
                                       C.byref(slot), C.byref(gen))
        if rc == _TIMEOUT:
            raise TimeoutError(f"no free ring slot for {owner!r} within {timeout}s")
        return RingLease(slot.value, gen.value, owner)

    def release(self, slot_id: int, generation: int, owner: str) -> None:
        rc = self._lib.ab_ring_release(self._h, int(slot_id), C.c_longlong(generation), owner.encode())
        if rc == _PENDING:
            raise RuntimeError("ring slot still has pending readers")
        if rc != _OK:
            raise RuntimeError("stale or duplicate ring lease release")

    def register_readers(self, lease: RingLease, readers: Iterable[str]) -> bool:
        names = [str(r) for r in readers]
        if not names:
            raise ValueError("at least one reader is required")
        rc = self._lib.ab_ring_register_readers(self._h, lease.slot_id, C.c_longlong(lease.generation),
                                                lease.owner.encode(), "\n".join(names).encode())
        if rc == _ALREADY_REG:
            raise RuntimeError("reader audience is already frozen for this lease")
        if rc == _STALE:
            raise RuntimeError("stale ring lease")
        return rc == _OK

    def reader_pending(self, lease: RingLease, reader: str) -> bool:
        return bool(self._lib.ab_ring_reader_pending(self._h, lease.slot_id, C.c_longlong(lease.generation),
                                                     lease.owner.encode(), reader.encode()))

    def release_reader(self, lease: RingLease, reader: str) -> bool:
        """Acknowledge one reader.  Returns True when this freed the slot."""
        freed = C.c_int()
        rc = self._lib.ab_ring_release_reader(self._h, lease.slot_id, C.c_longlong(lease.generation),
                                              lease.owner.encode(), reader.encode(), C.byref(freed))
        if rc == _NOT_READER:
            raise RuntimeError(f"{reader!r} is not a registered reader of this lease")
        if rc == _STALE:
            raise RuntimeError("stale ring lease")
        return bool(freed.value)

    def release_acknowledged(self, slot_id: int, generation: int, owner: str) -> bool:
        """Idempotent release: True when freed now, False when it was already acknowledged."""
        rc = self._lib.ab_ring_release_acknowledged(self._h, int(slot_id), C.c_longlong(generation), owner.encode())
        if rc == _OK:
            return True
        if rc == _ALREADY_ACK:
            return False
        if rc == _PENDING:
            raise RuntimeError("ring slot still has pending readers")
        raise RuntimeError("stale ring lease")
