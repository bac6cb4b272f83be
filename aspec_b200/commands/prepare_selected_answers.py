"""``select-answers``: from a corpus with several candidate answers per prompt (``candidates: [{"content", "score"}]``)
keep one answer per prompt by a selection rule and emit ordinary conversations
(reference: aspec/commands/prepare_selected_answers.py)."""
from __future__ import annotations

import argparse
import json
import sys


def select(row: dict, rule: str):
    cands = row.get("candidates") or []
    if not cands:
        return None
    if rule == "best_score":
        return max(cands, key=lambda c: (c.get("score", float("-inf")), -len(c.get("content", ""))))
    if rule == "shortest":
        return min(cands, key=lambda c: len(c.get("content", "")))
    if rule == "first":
        return cands[0]
    raise ValueError(f"unknown selection rule {rule!r}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 select-answers", description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--rule", default="best_score", choices=["best_score", "shortest", "first"])
    ap.add_argument("--min-score", type=float)
    a = ap.parse_args(argv)
    from aspec_b200.data.dataset import read_rows
    kept = dropped = 0
    with open(a.output, "w") as f:
        for row in read_rows(a.input):
            c = select(row, a.rule)
            if c is None or (a.min_score is not None and c.get("score", float("-inf")) < a.min_score):
                dropped += 1
                continue
            msgs = list(row.get("prompt") or row.get("messages") or [])
            msgs.append({"role": "assistant", "content": c["content"], **({"reasoning_content": c["reasoning_content"]}
                                                                         if c.get("reasoning_content") else {})})
            f.write(json.dumps({"id": row.get("id"), "conversations": msgs}, ensure_ascii=False) + "\n")
            kept += 1
    print(json.dumps({"output": a.output, "kept": kept, "dropped": dropped, "rule": a.rule}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
