"""Analytical acceptance statistics for block drafts (no host synchronisation).

``tau = 1 + sum_j prod_{i<=j} alpha_i`` is the expected accepted length including the Target's
bonus token; a fully masked block contributes nothing.  (aspec/models/ops/acceptance.py)
"""
from __future__ import annotations

import torch


def acceptance_statistics(accept_rate: torch.Tensor, eval_mask: torch.Tensor) -> torch.Tensor:
    """``[n_blocks, bs]`` inputs -> ``[2, bs + 1]`` (numerators; denominators), last column = tau."""
    if accept_rate.shape != eval_mask.shape or accept_rate.ndim != 2:
        raise ValueError("Acceptance and supervision must have matching [blocks, positions] shapes")
    mask = eval_mask.detach().float()
    alpha = accept_rate.detach().float() * mask
    valid = mask.bool().any(-1)
    tau = 1.0 + alpha.cumprod(-1).sum(-1)
    num = torch.cat((alpha.sum(0), (tau * valid).sum().reshape(1)))
    den = torch.cat((mask.sum(0), valid.sum().float().reshape(1)))
    return torch.stack((num, den))


def acceptance_components(stats: torch.Tensor) -> dict:
    keys = [f"accept_rate@{i}" for i in range(stats.shape[1] - 1)] + ["tau_probabilistic"]
    return {k: (stats[0, i], stats[1, i]) for i, k in enumerate(keys)}
