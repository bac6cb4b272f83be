"""Debug dumps of one training step: the batch, the loss terms and per-parameter gradient norms of a chosen step
are written to ``<run>/dumps/step-N-rankR.pt`` so that two runs (or two frameworks) can be compared offline
(reference: aspec/utils/train_dump.py)."""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch


def _cpu(value: Any) -> Any:
    if torch.is_tensor(value):
        return value.detach().to("cpu", copy=True)
    if isinstance(value, dict):
        return {k: _cpu(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_cpu(v) for v in value)
    return value


def dump_step(run_dir: str, step: int, rank: int, *, batch: Optional[Dict[str, Any]] = None, outputs: Any = None,
              model: Optional[torch.nn.Module] = None, max_tensor_elems: int = 1 << 22,
              grad_norms: Optional[Dict[str, float]] = None) -> str:
    """``grad_norms`` overrides the norms read from ``model`` (a trainer whose optimizer step clears the gradients
    captures them before the step)."""
    os.makedirs(os.path.join(run_dir, "dumps"), exist_ok=True)
    record: Dict[str, Any] = {"step": step, "rank": rank}
    if batch is not None:
        record["batch"] = {k: (_cpu(v) if not torch.is_tensor(v) or v.numel() <= max_tensor_elems
                               else {"shape": tuple(v.shape), "dtype": str(v.dtype), "norm": float(v.float().norm())})
                           for k, v in batch.items()}
    if outputs is not None:
        record["outputs"] = _cpu(outputs)
    if model is not None:
        grads = {}
        for name, p in model.named_parameters():
            g = getattr(p, "main_grad", None) if getattr(p, "main_grad_touched", False) else p.grad
            if g is not None:
                grads[name] = float(g.float().norm())
        record["grad_norms"] = grads if grad_norms is None else dict(grad_norms)
        record["param_norms"] = {n: float(p.detach().float().norm()) for n, p in model.named_parameters()}
    path = os.path.join(run_dir, "dumps", f"step-{step}-rank{rank}.pt")
    torch.save(record, path)
    return path
