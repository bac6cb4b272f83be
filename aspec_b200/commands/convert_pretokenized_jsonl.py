"""``convert-data``: conversations ``.jsonl`` -> pre-tokenised ``.jsonl`` (``input_ids`` + run-length ``packed_loss_mask``)
so that training start-up skips tokenisation (reference: aspec/commands/convert_pretokenized_jsonl.py)."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 convert-data", description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--tokenizer", required=True, help="local tokenizer directory")
    ap.add_argument("--chat-template", default="qwen")
    ap.add_argument("--max-seq-length", type=int, default=4096)
    ap.add_argument("--last-turn-loss-only", action="store_true")
    a = ap.parse_args(argv)
    from aspec_b200.data.dataset import load_training_samples
    report: dict = {}
    samples = load_training_samples(a.input, {"tokenizer_path": a.tokenizer, "chat_template": a.chat_template,
                                              "max_seq_length": a.max_seq_length,
                                              "last_turn_loss_only": True if a.last_turn_loss_only else None}, report=report)
    with open(a.output, "w") as f:
        for i, s in enumerate(samples):
            f.write(json.dumps({"data_id": s.get("data_id", f"sample_{i:08d}"), "input_ids": s["input_ids"].tolist(),
                                "packed_loss_mask": s["packed_loss_mask"]}) + "\n")
    print(json.dumps({"output": a.output, "samples": len(samples), **report}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
