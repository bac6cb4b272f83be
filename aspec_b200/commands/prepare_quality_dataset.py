"""``prepare-data``: deterministic train / held-out split of a conversation corpus with de-duplication and length
admission, writing ``train.jsonl``, ``eval.jsonl`` and a ``manifest.json`` with content hashes
(reference: aspec/commands/prepare_quality_dataset.py)."""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys


def _key(row: dict) -> str:
    msgs = row.get("conversations") or row.get("messages") or []
    return hashlib.sha256(json.dumps([[m.get("role", m.get("from")), m.get("content", m.get("value"))] for m in msgs],
                                     ensure_ascii=False).encode()).hexdigest()


def split_corpus(rows, eval_fraction: float, seed: int, min_turns: int = 2, max_chars: int = 0):
    seen, train, held = set(), [], []
    stats = {"seen": 0, "duplicates": 0, "too_short": 0, "too_long": 0}
    for row in rows:
        stats["seen"] += 1
        msgs = row.get("conversations") or row.get("messages") or []
        if len(msgs) < min_turns or not any((m.get("role", m.get("from")) in ("assistant", "gpt")) for m in msgs):
            stats["too_short"] += 1
            continue
        if max_chars and sum(len(str(m.get("content", m.get("value", "")))) for m in msgs) > max_chars:
            stats["too_long"] += 1
            continue
        k = _key(row)
        if k in seen:
            stats["duplicates"] += 1
            continue
        seen.add(k)
        # the split depends only on content and seed: re-running on a grown corpus never moves old rows
        bucket = int(hashlib.sha256(f"{seed}:{k}".encode()).hexdigest()[:8], 16) / 0xFFFFFFFF
        (held if bucket < eval_fraction else train).append(row)
    return train, held, stats


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 prepare-data", description=__doc__)
    ap.add_argument("--input", required=True, nargs="+")
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--eval-fraction", type=float, default=0.02)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-chars", type=int, default=0)
    a = ap.parse_args(argv)
    from aspec_b200.data.dataset import read_rows
    rows = [r for p in a.input for r in read_rows(p)]
    train, held, stats = split_corpus(rows, a.eval_fraction, a.seed, max_chars=a.max_chars)
    os.makedirs(a.output_dir, exist_ok=True)
    manifest = {"inputs": a.input, "seed": a.seed, "eval_fraction": a.eval_fraction, **stats}
    for name, part in (("train", train), ("eval", held)):
        path = os.path.join(a.output_dir, f"{name}.jsonl")
        with open(path, "w") as f:
            for r in part:
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
        manifest[name] = {"path": path, "rows": len(part), "sha256": hashlib.sha256(open(path, "rb").read()).hexdigest()}
    with open(os.path.join(a.output_dir, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=2)
    print(json.dumps(manifest, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
