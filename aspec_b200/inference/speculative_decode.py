"""Greedy speculative decoding with block proposals: the decode loop the reference gets from its serving engine
(aspec/inference/engine/sgl_engine_decode.py:39-424, train-with-decode and ``evaluate``), here on the in-framework Target.

One Target pass per round.  The pass over ``accepted + proposal`` verifies the proposal (the longest prefix on which the
Draft agrees with the Target's own greedy choice is accepted, and the Target's token after it comes for free) and, in the
same pass, yields the captured-layer features of every accepted token but the last - which is all the next proposal
needs, because a block anchored at the last token attends the context BEFORE its anchor.  The generated text is exactly
the Target's greedy continuation whatever the Draft proposes; the Draft only decides how many tokens a pass yields.

This is an evaluation loop, not a serving engine: there is no KV cache, every pass recomputes the prefix.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


@torch.no_grad()
def greedy_generate(target, prompt_ids: torch.Tensor, max_new_tokens: int, eos_token_id: Optional[int] = None) -> List[int]:
    """Plain greedy decoding with the Target alone (one pass per token): the oracle of ``speculative_generate``."""
    seq = [int(t) for t in prompt_ids.reshape(-1)]
    n0 = len(seq)
    dev = next(target.parameters()).device
    while len(seq) - n0 < max_new_tokens:
        out = target.prefill(torch.tensor(seq, device=dev), [len(seq)], [], want_logits=True)
        tok = int(out["logits"][-1].float().argmax())
        seq.append(tok)
        if eos_token_id is not None and tok == eos_token_id:
            break
    return seq[n0:]


@torch.no_grad()
def speculative_generate(target, consumer, prompt_ids: torch.Tensor, layer_ids: Sequence[int], *, max_new_tokens: int,
                         eos_token_id: Optional[int] = None) -> dict:
    """``consumer`` is a ``draft_artifact.BlockDraftConsumer``.  Returns the new tokens, the accepted Draft tokens of every
    round, the mean accepted length ``tau`` (tokens per Target pass) and the number of Target passes."""
    dev = next(target.parameters()).device
    lm_head = target.lm_head.detach()
    seq = [int(t) for t in prompt_ids.reshape(-1)]
    n0 = len(seq)
    per_round: List[int] = []
    passes = 1
    out = target.prefill(torch.tensor(seq, device=dev), [len(seq)], list(layer_ids), want_logits=True)
    feats = out["hidden_states"]                                       # [L, K * D]: features of every prompt token
    seq.append(int(out["logits"][-1].float().argmax()))                # the Target's first token
    width = feats.shape[-1]
    done = eos_token_id is not None and seq[-1] == eos_token_id
    while not done and len(seq) - n0 < max_new_tokens:
        known = len(seq) - 1                                           # every token but the anchor has features
        padded = torch.cat([feats[:known], feats.new_zeros(1, width)])[None]
        ids = torch.tensor(seq, device=dev)[None]
        proposal = consumer.propose(ids, padded, lm_head_weight=lm_head)["token_ids"].reshape(-1)[: consumer.block_size - 1]
        proposal = [int(t) for t in proposal]
        trial = seq + proposal
        out = target.prefill(torch.tensor(trial, device=dev), [len(trial)], list(layer_ids), want_logits=True)
        passes += 1
        greedy = out["logits"][len(seq) - 1:].float().argmax(-1).tolist()        # Target's choice after seq, seq+p1, ...
        n = 0
        while n < len(proposal) and proposal[n] == greedy[n]:
            n += 1
        new = proposal[:n] + [greedy[n]]
        if eos_token_id is not None and eos_token_id in new:
            new = new[: new.index(eos_token_id) + 1]
            done = True
        room = max_new_tokens - (len(seq) - n0)
        new = new[:room]
        per_round.append(min(n, len(new)))
        seq += new
        feats = out["hidden_states"][: len(seq) - 1]                   # valid: their inputs were all accepted tokens
    tokens = seq[n0:]
    return {"tokens": tokens, "accepted_per_round": per_round, "target_passes": passes,
            "tau": (len(tokens) - 1) / max(len(per_round), 1) if per_round else 1.0,
            "mean_accepted_draft_tokens": sum(per_round) / max(len(per_round), 1)}
