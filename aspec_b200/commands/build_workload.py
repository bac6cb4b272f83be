"""``build-workload``: deterministic pre-tokenised benchmark workloads.

``fixed``: ``--rows`` documents of exactly ``--sequence-length`` uniformly random token ids (seeded), every position
after ``--prompt-tokens`` supervised - the Draft-only and scheduler benchmarks' input.  ``mixed``: documents cut from
a pre-tokenised source to a cycle of lengths (``--lengths``, ``--repetitions``), ids and masks preserved - the
packing / scheduler workload.  Both write ``.jsonl`` rows ``{data_id, input_ids, packed_loss_mask, seq_len,
loss_tokens}`` and print a manifest with the file's SHA-256 (reference: tools/build_fixed_token_workload.py,
tools/build_mixed_length_workload.py; the reference also writes parquet)."""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _write(rows, destination: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(destination)), exist_ok=True)
    tmp = destination + ".partial"
    with open(tmp, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    os.replace(tmp, destination)


def build_fixed(destination: str, *, sequence_length: int, rows: int, seed: int, min_token_id: int, max_token_id: int,
                prompt_tokens: int = 0) -> dict:
    import numpy as np
    from aspec_b200.data.utils import pack_loss_mask
    import torch
    if sequence_length < 2 or rows < 1:
        raise ValueError("sequence_length >= 2 and rows >= 1 are required")
    if min_token_id < 0 or max_token_id <= min_token_id:
        raise ValueError("token ID range must be non-negative and non-empty")
    if not 0 <= prompt_tokens < sequence_length:
        raise ValueError("prompt_tokens must lie inside the sequence")
    rng = np.random.default_rng(seed)
    mask = torch.cat([torch.zeros(prompt_tokens), torch.ones(sequence_length - prompt_tokens)])
    packed = pack_loss_mask(mask)

    def gen():
        for i in range(rows):
            ids = rng.integers(min_token_id, max_token_id, size=sequence_length, dtype=np.int64)
            yield {"data_id": f"fixed_{sequence_length}_{i:08d}", "input_ids": ids.tolist(), "packed_loss_mask": packed,
                   "seq_len": sequence_length, "loss_tokens": sequence_length - prompt_tokens}

    _write(gen(), destination)
    return {"generator": "aspec_b200.fixed-token-workload/v1", "destination": destination, "rows": rows,
            "sequence_length": sequence_length, "seed": seed, "min_token_id": min_token_id,
            "max_token_id_exclusive": max_token_id, "prompt_tokens": prompt_tokens, "sha256": _sha256(destination)}


def build_mixed(source: str, destination: str, *, lengths, repetitions: int) -> dict:
    import torch
    from aspec_b200.data.utils import pack_loss_mask, unpack_loss_mask
    lengths = [int(v) for v in lengths]
    if not lengths or min(lengths) <= 0 or repetitions <= 0:
        raise ValueError("lengths and repetitions must be positive")
    want = repetitions * len(lengths)
    src = []
    with open(source) as f:
        for line in f:
            if line.strip():
                src.append(json.loads(line))
            if len(src) >= want:
                break
    if not src:
        raise ValueError("source has no JSONL rows")
    out = []
    for rep in range(repetitions):
        for off, n in enumerate(lengths):
            row = src[(rep * len(lengths) + off) % len(src)]
            ids = row["input_ids"]
            mask = (torch.tensor(row["loss_mask"]) if "loss_mask" in row
                    else unpack_loss_mask(row["packed_loss_mask"], len(ids)))
            if len(ids) < n or mask.numel() < n:
                raise ValueError(f"source row is shorter than requested length {n}")
            m = mask[:n].float()
            out.append({"data_id": f"mixed_{rep:04d}_{off:02d}_{n}", "input_ids": ids[:n], "packed_loss_mask": pack_loss_mask(m),
                        "seq_len": n, "loss_tokens": int(m.sum())})
    _write(out, destination)
    return {"generator": "aspec_b200.mixed-length-workload/v1", "destination": destination, "rows": len(out),
            "lengths": lengths, "repetitions": repetitions, "source_sha256": _sha256(source), "sha256": _sha256(destination)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 build-workload", description=__doc__)
    sub = ap.add_subparsers(dest="kind", required=True)
    fx = sub.add_parser("fixed")
    fx.add_argument("destination")
    fx.add_argument("--sequence-length", type=int, default=4096)
    fx.add_argument("--rows", type=int, default=1024)
    fx.add_argument("--seed", type=int, default=0)
    fx.add_argument("--min-token-id", type=int, default=0)
    fx.add_argument("--max-token-id", type=int, default=150000)
    fx.add_argument("--prompt-tokens", type=int, default=0)
    mx = sub.add_parser("mixed")
    mx.add_argument("source")
    mx.add_argument("destination")
    mx.add_argument("--lengths", default="512,768,1024,1536,2048,3072,3584,4096")
    mx.add_argument("--repetitions", type=int, default=8)
    a = ap.parse_args(argv)
    if a.kind == "fixed":
        man = build_fixed(a.destination, sequence_length=a.sequence_length, rows=a.rows, seed=a.seed,
                          min_token_id=a.min_token_id, max_token_id=a.max_token_id, prompt_tokens=a.prompt_tokens)
    else:
        man = build_mixed(a.source, a.destination, lengths=a.lengths.split(","), repetitions=a.repetitions)
    print(json.dumps(man))
    return 0


if __name__ == "__main__":
    sys.exit(main())
