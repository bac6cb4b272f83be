"""Low-rank candidate retrieval head of EAGLE4: ``scores = up(down(h))`` with ``down: H -> r`` and ``up: r -> V``.

The head is trained in a stage of its own to reproduce the frozen Draft's top-k distribution; serving uses it to
pull a shortlist of token ids whose exact logits are then computed with the full head.  Before its first update it
is initialised to the best rank-``r`` approximation of the exact head (reference behaviour:
aspec/models/draft/eagle4.py:123-146).  The factorisation here is a hand-rolled randomised range finder so that the
workspace stays ``V x (r + oversample)`` instead of a full ``V x H`` singular basis.
"""
from __future__ import annotations

from typing import Tuple

import torch

CANDIDATE_MODULES = ("efficient_lm_head", "efficient_lm_head_down_proj")


def is_candidate_parameter(name: str) -> bool:
    return name.split(".", 1)[0] in CANDIDATE_MODULES


def stage_trains(name: str, stage: str) -> bool:
    """Which parameters a stage updates: ``candidate_head`` trains the two projections only, ``draft`` the rest."""
    return is_candidate_parameter(name) == (stage == "candidate_head")


@torch.no_grad()
def low_rank_factors(weight: torch.Tensor, rank: int, *, oversample: int = 16, power_iterations: int = 2,
                     generator: torch.Generator | None = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(down [rank, H], up [V, rank])`` with ``up @ down`` the rank-``rank`` truncation of ``weight [V, H]``.

    Randomised subspace iteration: sketch the row space with a Gaussian test matrix, sharpen it with a few
    orthonormalised power iterations, then take the exact SVD of the small projected matrix.
    """
    W = weight.to(torch.float32)
    V, H = W.shape
    width = min(rank + oversample, V, H)
    omega = torch.randn(H, width, dtype=W.dtype, device=W.device, generator=generator)
    basis, _ = torch.linalg.qr(W @ omega)                      # [V, width], spans the dominant column space
    for _ in range(power_iterations):
        z, _ = torch.linalg.qr(W.T @ basis)                    # [H, width]
        basis, _ = torch.linalg.qr(W @ z)
    small = basis.T @ W                                        # [width, H]
    u_small, sigma, vh = torch.linalg.svd(small, full_matrices=False)
    keep = min(rank, width)
    up = (basis @ u_small[:, :keep]) * sigma[:keep]            # [V, keep], singular values folded in
    down = vh[:keep]                                           # [keep, H]
    if keep < rank:                                            # degenerate tiny heads: pad with zeros
        up = torch.cat([up, up.new_zeros(V, rank - keep)], 1)
        down = torch.cat([down, down.new_zeros(rank - keep, H)], 0)
    return down, up


@torch.no_grad()
def shortlist_logits(head_weight: torch.Tensor, hidden: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """Exact logits ``hidden . head_weight[id]`` for every id of each row's shortlist: ``[..., k]``."""
    rows = head_weight[token_ids]                              # [..., k, H]
    return torch.einsum("...kh,...h->...k", rows.float(), hidden.float()).to(hidden.dtype)
