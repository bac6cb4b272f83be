"""Which implementation of an op actually ran in this process.

The plan states which kernel each subsystem should use; the dispatchers in ``ops/`` count what they really launched
(``note("attention", "tcgen05_interval_flash")``) and the run's evidence records the counts beside the plan's decision,
so a silent fallback is visible in ``evidence.json`` (the reference carries per-layer attention observations to its
evidence the same way: aspec/models/ops/direct_cp.py:990-1023, aspec/training/trainer.py:569-629)."""
from __future__ import annotations

from collections import defaultdict
from typing import Dict

_counts: Dict[str, Dict[str, int]] = defaultdict(lambda: defaultdict(int))


def note(subsystem: str, implementation: str) -> None:
    _counts[subsystem][implementation] += 1


def snapshot() -> Dict[str, Dict[str, int]]:
    return {s: dict(impls) for s, impls in _counts.items()}


def reset() -> None:
    _counts.clear()
