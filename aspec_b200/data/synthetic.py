"""Synthetic documents and Target features for benchmarks, tests and quick starts.

There is no network for datasets or checkpoints, so every shipped recipe can run on generated
data: token ids uniform over the vocabulary, document lengths log-uniform (or fixed), the loss mask
covering the final fraction of each document, and - for Draft-only runs that skip the Target - random
bf16 "captured layer" features of the right shape.  The per-row generator is seeded by
``(seed, row)`` so any rank can materialise any row without coordination (the reference's fixed-token
workload builder does the same: tools/build_fixed_token_workload.py:52-147).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterator, Optional

import numpy as np
import torch


@dataclass
class SyntheticSpec:
    vocab_size: int = 151936
    min_len: int = 256
    max_len: int = 4096
    length_distribution: str = "log_uniform"     # log_uniform | uniform | fixed
    loss_tail_fraction: float = 0.6              # final fraction of the document that is supervised
    seed: int = 0
    token_low: int = 0
    token_high: Optional[int] = None


def document_length(spec: SyntheticSpec, row: int) -> int:
    rng = np.random.default_rng(np.random.SeedSequence([spec.seed, row, 1]))
    if spec.length_distribution == "fixed" or spec.min_len == spec.max_len:
        return spec.max_len
    if spec.length_distribution == "uniform":
        return int(rng.integers(spec.min_len, spec.max_len + 1))
    u = rng.random()
    return int(round(math.exp(math.log(spec.min_len) + u * (math.log(spec.max_len) - math.log(spec.min_len)))))


def make_document(spec: SyntheticSpec, row: int) -> dict:
    """``{"data_id", "input_ids" int64 [L], "loss_mask" float32 [L], "packed_loss_mask" str}``."""
    n = document_length(spec, row)
    rng = np.random.default_rng(np.random.SeedSequence([spec.seed, row]))
    hi = spec.token_high or spec.vocab_size
    ids = torch.from_numpy(rng.integers(spec.token_low, hi, size=n, dtype=np.int64))
    n_sup = max(int(round(n * spec.loss_tail_fraction)), 0)
    mask = torch.zeros(n, dtype=torch.float32)
    if n_sup:
        mask[n - n_sup:] = 1.0
    return {"data_id": f"synthetic-{spec.seed}-{row}", "input_ids": ids, "loss_mask": mask,
            "packed_loss_mask": f"{n - n_sup},{n_sup}" if n_sup else f"{n}", "seq_len": n}


def synthetic_features(n_tokens: int, n_layers: int, hidden: int, row: int, seed: int = 0,
                       dtype=torch.bfloat16, pin: bool = False) -> dict:
    """Random stand-ins for captured Target layers ``[T, K*Dt]`` and the post-norm last hidden ``[T, Dt]``."""
    g = torch.Generator().manual_seed((seed * 1000003 + row) % (2 ** 63))
    hs = torch.randn(n_tokens, n_layers * hidden, generator=g, dtype=torch.float32).to(dtype)
    last = torch.randn(n_tokens, hidden, generator=g, dtype=torch.float32).to(dtype)
    if pin and torch.cuda.is_available():
        hs, last = hs.pin_memory(), last.pin_memory()
    return {"hidden_states": hs, "last_hidden_states": last}


def iter_documents(spec: SyntheticSpec, start: int = 0, count: Optional[int] = None) -> Iterator[dict]:
    row = start
    while count is None or row < start + count:
        yield make_document(spec, row)
        row += 1


def mean_length(spec: SyntheticSpec, rows: int = 2048) -> float:
    return float(np.mean([document_length(spec, r) for r in range(rows)]))


def benchmark_documents(spec: SyntheticSpec, n_docs: int, per_update: int, rank: int = 0) -> list:
    """The benchmark's document pool, identical in shape for every arm and rank.

    Document ``i`` has the length of row ``i`` of ``spec`` on every rank (so per-GPU work does not depend on the number of
    GPUs); ranks above 0 draw their own token ids.  The documents are then dealt to the updates (``per_update``
    consecutive pool entries each) by length, serpentine over the sorted list, so that every update carries about the
    same number of tokens.  Each entry is ``make_document``'s dictionary plus ``"row"`` (a per-rank seed for features).
    """
    docs = []
    for i in range(n_docs):
        doc = make_document(spec, i)
        row = rank * 100003 + i
        if rank > 0:
            g = torch.Generator().manual_seed(row)
            doc["input_ids"] = torch.randint(0, spec.vocab_size, (doc["seq_len"],), generator=g, dtype=torch.int64)
        doc["row"] = row
        docs.append(doc)
    groups = max(n_docs // max(per_update, 1), 1)
    if groups > 1 and n_docs % groups == 0:
        order = sorted(range(n_docs), key=lambda i: -docs[i]["seq_len"])
        buckets = [[] for _ in range(groups)]
        for j, i in enumerate(order):
            g = j % groups
            buckets[g if (j // groups) % 2 == 0 else groups - 1 - g].append(i)
        docs = [docs[i] for b in buckets for i in b]
    return docs
