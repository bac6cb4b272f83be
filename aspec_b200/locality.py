"""Per-node apportionment of ready credits and sample budgets: when Target engines and Draft trainers live on
several nodes, each node's producers may only run ahead by its share of the ready pool, proportional to the
consumers it feeds (largest-remainder rounding, never zero for an active node)
(reference: aspec/locality.py:22-93)."""
from __future__ import annotations

from typing import Dict, Mapping


def apportion(total: int, weights: Mapping[str, float], minimum: int = 1) -> Dict[str, int]:
    """Split ``total`` units over keys in proportion to ``weights`` (largest remainder; active keys get >= minimum)."""
    active = {k: float(w) for k, w in weights.items() if w > 0}
    if not active:
        return {k: 0 for k in weights}
    if total < minimum * len(active):
        raise ValueError(f"cannot give {len(active)} nodes at least {minimum} of {total} units")
    spare = total - minimum * len(active)
    norm = sum(active.values())
    exact = {k: spare * w / norm for k, w in active.items()}
    out = {k: minimum + int(v) for k, v in exact.items()}
    left = total - sum(out.values())
    for k in sorted(active, key=lambda k: (exact[k] - int(exact[k]), active[k], k), reverse=True)[:left]:
        out[k] += 1
    return {k: out.get(k, 0) for k in weights}


def node_ready_credits(ready_pool_capacity: int, trainers_per_node: Mapping[str, int]) -> Dict[str, int]:
    return apportion(ready_pool_capacity, trainers_per_node)


def node_sample_budgets(samples_per_update: int, engines_per_node: Mapping[str, int]) -> Dict[str, int]:
    return apportion(samples_per_update, engines_per_node, minimum=0 if samples_per_update < len(engines_per_node) else 1)
