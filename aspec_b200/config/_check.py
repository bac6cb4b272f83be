"""Tiny typed-value checkers shared by the draft policy resolvers."""
from __future__ import annotations

import math
from typing import Any, Mapping


def pos_int(raw: Mapping, key: str, default: Any = None, *, what: str = "Draft") -> int:
    value = raw.get(key, default)
    if value is None:
        value = default
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ValueError(f"{what} {key} must be a positive integer")
    return value


def nonneg_number(raw: Mapping, key: str, default: float, *, what: str = "Draft",
                  positive: bool = False) -> float:
    value = raw.get(key, default)
    if value is None:
        value = default
    bad = (isinstance(value, bool) or not isinstance(value, (int, float))
           or not math.isfinite(value) or value < 0 or (positive and value == 0))
    if bad:
        kind = "positive" if positive else "non-negative"
        raise ValueError(f"{what} {key} must be finite and {kind}")
    return float(value)


def boolean(raw: Mapping, key: str, default: bool, *, what: str = "Draft") -> bool:
    value = raw.get(key, default)
    if not isinstance(value, bool):
        raise ValueError(f"{what} {key} must be boolean")
    return value
