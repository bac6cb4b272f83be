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


# -- generation with cached keys / values, several sequences per pass ----------------------------------------------------
def filter_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """Log-weights of the sampling distribution: temperature, then top-k, then nucleus (top-p) filtering; removed entries
    are ``-inf``.  ``temperature <= 0`` means greedy and returns the logits untouched."""
    x = logits.float()
    if temperature <= 0:
        return x
    x = x / float(temperature)
    if top_k and 0 < top_k < x.shape[-1]:
        kth = x.topk(int(top_k), -1).values[..., -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    if 0.0 < top_p < 1.0:
        sorted_x, order = x.sort(-1, descending=True)
        probs = torch.softmax(sorted_x, -1)
        before = probs.cumsum(-1) - probs                      # mass of the strictly more likely tokens
        drop = before >= top_p                                 # the most likely token always stays
        x = x.masked_fill(torch.zeros_like(drop).scatter(-1, order, drop), float("-inf"))
    return x


def _wrap64(value: int) -> int:
    """A 64-bit constant as the signed integer an int64 tensor holds."""
    value &= (1 << 64) - 1
    return value - (1 << 64) if value >= 1 << 63 else value


def keyed_uniform(seed: int, positions: torch.Tensor, width: int) -> torch.Tensor:
    """Uniform numbers in (0, 1), ``[len(positions), width]``, that are a pure function of ``(seed, position, column)``:
    a counter-based generator (the SplitMix64 finaliser over ``seed``, position and column, in wrapping int64
    arithmetic).  A token position therefore meets the same noise whenever and with whatever neighbours it is drawn - in
    a verify pass over a Draft block, one token at a time, before or after a restart."""
    dev = positions.device
    col = torch.arange(width, device=dev, dtype=torch.int64)[None]
    z = col * _wrap64(0x9E3779B97F4A7C15) + (positions.to(torch.int64)[:, None] + 1) * _wrap64(0xD1B54A32D192ED03) \
        + _wrap64(int(seed) * 0x2545F4914F6CDD1D + 0x632BE59BD9B4E019)
    for shift, mult in ((30, 0xBF58476D1CE4E5B9), (27, 0x94D049BB133111EB)):
        z = (z ^ ((z >> shift) & ((1 << (64 - shift)) - 1))) * _wrap64(mult)
    z = z ^ ((z >> 31) & ((1 << 33) - 1))
    top = (z >> 40) & ((1 << 24) - 1)                         # 24 high bits: exactly representable in float32
    return (top.to(torch.float32) + 0.5) / float(1 << 24)


def sample_tokens(logits: torch.Tensor, temperature: float = 1.0, top_k: int = -1, top_p: float = 1.0,
                  seed: int = 0, first_position: int = 0) -> torch.Tensor:
    """One token per row of ``logits [m, V]``; row ``i`` is the sequence's new token number ``first_position + i``.
    Sampling is Gumbel-max on the filtered log-weights with noise keyed by ``(seed, token number)``: what a sequence
    samples at a position depends on its logits there and on nothing else."""
    x = filter_logits(logits, temperature, top_k, top_p)
    if temperature <= 0:
        return x.argmax(-1)
    positions = torch.arange(first_position, first_position + x.shape[0], device=x.device)
    u = keyed_uniform(seed, positions, x.shape[-1])
    return (x - torch.log(-torch.log(u))).argmax(-1)


@torch.no_grad()
def batched_generate(target, prompts: Sequence[torch.Tensor], *, max_new_tokens: Sequence[int], min_new_tokens: int = 0,
                     stop_token_ids: Sequence[int] = (), temperature: float = 1.0, top_k: int = -1, top_p: float = 1.0,
                     seeds: Optional[Sequence[int]] = None, consumer=None, layer_ids: Sequence[int] = ()) -> List[dict]:
    """Continue every prompt with the Target's own tokens; all sequences share each Target pass and keep their keys and
    values in one cache (``DenseTarget.extend``), so a pass costs the new tokens only.

    With ``consumer`` (a ``draft_artifact.BlockDraftConsumer``) a pass verifies a Draft block per sequence: the Target's
    token is drawn at every proposed position, the proposal is accepted as long as it equals those draws, and the first
    draw that differs is kept - every kept token is a draw from the Target's distribution given its prefix, and the noise
    of a draw is keyed by the sequence's seed and the token's number (``sample_tokens``), so the text is THE SAME with any
    Draft, with none, and in any batch; the Draft only changes how many tokens a pass yields.  Stop tokens are masked out
    until ``min_new_tokens`` tokens exist.  ``seeds[r]`` is sequence ``r``'s noise seed.

    Returns per sequence ``{"tokens", "target_passes", "accepted_per_round", "stopped"}``."""
    dev = target.lm_head.device
    R = len(prompts)
    if R == 0:
        return []
    block = int(consumer.block_size) if consumer is not None else 1
    budget = [int(m) for m in max_new_tokens]
    capacity = max(int(p.numel()) + b for p, b in zip(prompts, budget)) + block
    cache = target.new_decode_cache(R, capacity)
    noise_seeds = [int(seeds[r]) if seeds is not None else r for r in range(R)]
    stops = [int(t) for t in (stop_token_ids or ())]
    # ranks of a tensor-parallel Target take rank 0's draws and proposals, so that all of them run the same passes
    agree = getattr(target, "agree", lambda t: t)
    lm_head = target.lm_head.detach()
    capture = list(layer_ids) if consumer is not None else []
    seqs = [[int(t) for t in p.reshape(-1)] for p in prompts]
    n0 = [len(s) for s in seqs]
    feats: List[Optional[torch.Tensor]] = [None] * R
    out = [{"tokens": [], "target_passes": 0, "accepted_per_round": [], "stopped": "length"} for _ in range(R)]
    active = [r for r in range(R) if budget[r] > 0]

    def draw(r: int, logits: torch.Tensor, already: int) -> List[int]:
        """Target tokens at consecutive positions of sequence ``r``; position ``i`` has ``already + i`` new tokens before it."""
        if stops and min_new_tokens > 0:
            logits = logits.clone()
            for i in range(logits.shape[0]):
                if already + i < min_new_tokens:
                    logits[i, stops] = float("-inf")
        return agree(sample_tokens(logits, temperature, top_k, top_p, noise_seeds[r], already)).tolist()

    def keep(r: int, new: List[int]) -> None:
        room = budget[r] - (len(seqs[r]) - n0[r])
        new = new[:room]
        for i, t in enumerate(new):
            if t in stops:
                new = new[: i + 1]
                out[r]["stopped"] = "stop_token"
                break
        seqs[r] += new
        if out[r]["stopped"] == "stop_token" or len(seqs[r]) - n0[r] >= budget[r]:
            active.remove(r)

    # the prompts: one pass, the first new token of every sequence
    first = target.extend(cache, [torch.tensor(seqs[r]) if r in active else torch.empty(0, dtype=torch.long) for r in range(R)], capture)
    for r in list(active):
        lo, hi = first["offsets"][r], first["offsets"][r + 1]
        cache.accept(r, hi - lo)
        if consumer is not None:
            feats[r] = first["hidden_states"][lo:hi]
        out[r]["target_passes"] += 1
        keep(r, draw(r, first["logits"][hi - 1:hi], 0))
    while active:
        trial = {}
        for r in active:
            proposal: List[int] = []
            if consumer is not None:
                known = len(seqs[r]) - 1                      # every token but the newest has features
                padded = torch.cat([feats[r][:known], feats[r].new_zeros(1, feats[r].shape[-1])])[None]
                ids = torch.tensor(seqs[r], device=dev)[None]
                proposal = [int(t) for t in agree(consumer.propose(ids, padded, lm_head_weight=lm_head)["token_ids"].reshape(-1)[: block - 1])]
                proposal = proposal[: max(budget[r] - (len(seqs[r]) - n0[r]) - 1, 0)]
            trial[r] = proposal
        step = target.extend(cache, [torch.tensor([seqs[r][-1]] + trial[r]) if r in trial else torch.empty(0, dtype=torch.long)
                                     for r in range(R)], capture)
        for r in list(active):
            lo, hi = step["offsets"][r], step["offsets"][r + 1]
            proposal = trial[r]
            drawn = draw(r, step["logits"][lo:hi], len(seqs[r]) - n0[r])
            n = 0
            while n < len(proposal) and proposal[n] == drawn[n]:
                n += 1
            cache.accept(r, 1 + n)                            # the newest token and the accepted proposals are cached now
            if consumer is not None:
                feats[r] = torch.cat([feats[r][: len(seqs[r]) - 1], step["hidden_states"][lo:lo + 1 + n]])
            out[r]["target_passes"] += 1
            if consumer is not None:
                out[r]["accepted_per_round"].append(n)
            keep(r, proposal[:n] + [drawn[n]])
    for r in range(R):
        out[r]["tokens"] = seqs[r][n0[r]:]
    return out
