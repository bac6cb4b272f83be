"""L1 distance between sampling-transformed Draft and Target distributions.

The DSpark objective can measure ``sum_v |p_draft(v) - p_target(v)|`` on the distributions a sampler would
actually draw from: temperature first, then the joint top-k / top-p support computed on the temperature-scaled
distribution; tokens outside the support get probability zero and the survivors are renormalised
(reference: aspec/models/ops/loss.py:56-91, aspec/models/dspark.py:596-609).  The support is discrete and carries
no gradient; the logits inside it do.

This path is only taken when a recipe sets a non-default ``dspark_l1_*`` temperature / top-p / top-k.  The logits
come from the tcgen05 GEMM (``ops.linear``) in row chunks, each chunk recomputed in backward, so at most
``chunk_rows x V`` fp32 values of each distribution exist at a time.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch.utils.checkpoint import checkpoint

from aspec_b200.ops.linear import linear

DEFAULT_SAMPLING = (1.0, 1.0, -1)


def sampling_logits(logits: torch.Tensor, sampling: Sequence = DEFAULT_SAMPLING) -> torch.Tensor:
    """Logits restricted to the sampler's support (``-inf`` outside).  ``sampling = (temperature, top_p, top_k)``.

    Order of ties: lower token id first (stable descending sort).  ``top_p`` keeps the shortest prefix of the sorted
    distribution whose mass before the token is ``<= top_p``; ``top_k`` keeps the first ``k`` sorted tokens; both
    are evaluated on the same temperature-scaled distribution and intersected.
    """
    temperature, top_p, top_k = float(sampling[0]), float(sampling[1]), int(sampling[2])
    if (temperature, top_p, top_k) == DEFAULT_SAMPLING:
        return logits
    if temperature <= 0:
        raise ValueError("sampling temperature must be positive")
    z = logits.float()
    if temperature != 1.0:
        z = (z - z.amax(dim=-1, keepdim=True)) / temperature
    V = z.shape[-1]
    use_k = 0 < top_k < V
    if top_p >= 1.0 and not use_k:
        return z
    ordered, order = z.sort(dim=-1, descending=True, stable=True)
    drop = torch.zeros_like(ordered, dtype=torch.bool)
    if top_p < 1.0:
        pr = ordered.softmax(dim=-1)
        drop = (pr.cumsum(dim=-1) - pr) > top_p
    if use_k:
        drop = drop | (torch.arange(V, device=z.device) >= top_k)
    mask = torch.zeros_like(drop).scatter(-1, order, drop)
    return z.masked_fill(mask, float("-inf"))


def l1_between(logits: torch.Tensor, target_logits: torch.Tensor, target_sampling=DEFAULT_SAMPLING,
               draft_sampling=DEFAULT_SAMPLING) -> torch.Tensor:
    p = torch.softmax(sampling_logits(logits, draft_sampling).float(), dim=-1)
    q = torch.softmax(sampling_logits(target_logits, target_sampling).float(), dim=-1)
    return (p - q).abs().sum(dim=-1)


def sampled_l1(hidden: torch.Tensor, lm_w: torch.Tensor, teacher_rows: torch.Tensor, *,
               prev_emb: Optional[torch.Tensor] = None, markov_w2: Optional[torch.Tensor] = None,
               target_sampling=DEFAULT_SAMPLING, draft_sampling=DEFAULT_SAMPLING, chunk_rows: int = 512) -> torch.Tensor:
    """Per-row L1 ``[R]`` (fp32, differentiable in ``hidden``, ``prev_emb`` and ``markov_w2``).

    ``hidden [R, D]`` Draft states, ``teacher_rows [R, D]`` the Target's last hidden state of each row (already
    gathered), ``lm_w [V, D]`` the frozen head, ``prev_emb [R, r]`` / ``markov_w2 [V, r]`` the Markov bias.
    """
    def one(h, t, pe):
        z = linear(h, lm_w).float()
        if pe is not None:
            z = z + linear(pe, markov_w2).float()
        with torch.no_grad():
            zt = linear(t, lm_w).float()
        return l1_between(z, zt, target_sampling, draft_sampling)

    out = []
    for lo in range(0, hidden.shape[0], chunk_rows):
        hi = min(lo + chunk_rows, hidden.shape[0])
        pe = prev_emb[lo:hi] if prev_emb is not None else None
        if torch.is_grad_enabled() and (hidden.requires_grad or (pe is not None and pe.requires_grad)):
            out.append(checkpoint(one, hidden[lo:hi], teacher_rows[lo:hi], pe, use_reentrant=False))
        else:
            out.append(one(hidden[lo:hi], teacher_rows[lo:hi], pe))
    return torch.cat(out) if out else hidden.new_zeros(0, dtype=torch.float32)
