"""Dataset preprocessing: conversations -> token ids + run-length loss masks, and the token-frequency vocabulary
mapping used by pruned-vocabulary EAGLE drafts (reference: aspec/data/preprocessing.py:67-427)."""
from __future__ import annotations

from collections import Counter
from typing import Any, Dict, Iterable, List, Optional, Sequence

import torch

from aspec_b200.data.parse import Parser, has_thinking_content, has_unbalanced_thinking_tags, normalize_conversation
from aspec_b200.data.utils import pack_loss_mask, unpack_loss_mask
from aspec_b200.models.vocab import build_vocab_mapping


def preprocess_conversations(parser: Parser, conversations: Iterable[Sequence[Dict[str, Any]]], max_length: int,
                             last_turn_loss_only: Optional[bool] = None, report: Optional[dict] = None) -> List[dict]:
    """One record per admitted conversation: ``{"input_ids", "packed_loss_mask", "source_index"}`` (its place in the
    input, so that the caller can name it after its source row).

    ``last_turn_loss_only=None`` decides per conversation: reasoning traces are only reproducible for the final
    turn (history turns lose their ``<think>`` blocks), so conversations with reasoning supervise the last turn.
    """
    out = []
    stats = Counter()
    for conv in conversations:
        stats["seen"] += 1
        try:
            msgs = normalize_conversation(conv)
        except ValueError:
            stats["rejected_malformed"] += 1
            continue
        if not any(m["role"] == "assistant" for m in msgs):
            stats["rejected_no_assistant"] += 1
            continue
        last_only = has_thinking_content(msgs) if last_turn_loss_only is None else bool(last_turn_loss_only)
        text = parser.format(msgs, last_turn_only=last_only)
        if has_unbalanced_thinking_tags(text):
            stats["rejected_unbalanced_thinking"] += 1
            continue
        ids, mask = parser.tokenize_with_loss_mask(text, max_length, last_only)
        if int(mask.sum()) == 0:
            stats["rejected_no_supervised_tokens"] += 1
            continue
        stats["admitted"] += 1
        stats["last_turn_only"] += int(last_only)
        out.append({"input_ids": ids, "packed_loss_mask": pack_loss_mask(mask), "source_index": stats["seen"] - 1})
    if report is not None:
        report.update(dict(stats))
    return out


def count_token_frequencies(samples: Iterable[dict]) -> Counter:
    """Frequencies of supervised tokens only (the draft head never has to produce prompt tokens)."""
    counts: Counter = Counter()
    for s in samples:
        ids = s["input_ids"].reshape(-1)
        mask = unpack_loss_mask(s["packed_loss_mask"], ids.numel(), dtype=torch.bool)
        vals, n = torch.unique(ids[mask], return_counts=True)
        counts.update(dict(zip(vals.tolist(), n.tolist())))
    return counts


def generate_vocab_mapping(samples: Iterable[dict], target_vocab_size: int, draft_vocab_size: int,
                           always_keep: Sequence[int] = ()):
    """``(d2t, t2d)`` for the ``draft_vocab_size`` most frequent supervised tokens (ties by id; padded with the
    lowest unused ids when the corpus has fewer distinct tokens)."""
    if not 0 < draft_vocab_size <= target_vocab_size:
        raise ValueError("draft_vocab_size must be in (0, target_vocab_size]")
    counts = count_token_frequencies(samples)
    chosen = list(dict.fromkeys(int(t) for t in always_keep))
    for tok, _ in sorted(counts.items(), key=lambda kv: (-kv[1], kv[0])):
        if len(chosen) >= draft_vocab_size:
            break
        if tok not in chosen and tok < target_vocab_size:
            chosen.append(tok)
    if len(chosen) < draft_vocab_size:
        have = set(chosen)
        chosen += [t for t in range(target_vocab_size) if t not in have][: draft_vocab_size - len(chosen)]
    selected = torch.tensor(sorted(chosen[:draft_vocab_size]), dtype=torch.long)
    return build_vocab_mapping(selected, target_vocab_size)
