"""Training-sample loading: a ``.jsonl`` / ``.json`` file of conversations (``{"conversations": [...]}`` or
``{"messages": [...]}``) or of pre-tokenised rows (``{"input_ids": [...], "loss_mask": [...]}``) becomes the
controller's sample list, with an identity-bound on-disk cache (reference: aspec/data/dataset.py:62-520).

The cache key covers everything that changes the tokens: file digest, tokenizer path, template, max length, loss
policy and the parser version, so a stale cache cannot be picked up after a recipe change.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, List, Mapping, Optional

import torch

from aspec_b200.data.parse import create_parser
from aspec_b200.data.preprocessing import preprocess_conversations
from aspec_b200.data.template import TEMPLATE_REGISTRY
from aspec_b200.data.utils import pack_loss_mask

PARSER_VERSION = "2"          # 2: every sample carries its data_id


def _file_digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def read_rows(path: str) -> List[dict]:
    with open(path) as f:
        if path.endswith(".jsonl"):
            return [json.loads(line) for line in f if line.strip()]
        data = json.load(f)
    return data if isinstance(data, list) else data.get("data", [])


def is_pretokenized(rows: List[dict]) -> bool:
    return bool(rows) and "input_ids" in rows[0]


def _from_pretokenized(rows: List[dict], max_length: int) -> List[dict]:
    out = []
    for i, r in enumerate(rows):
        ids = torch.tensor(r["input_ids"], dtype=torch.long)[:max_length]
        if "packed_loss_mask" in r:
            packed = r["packed_loss_mask"]
        else:
            mask = torch.tensor(r.get("loss_mask") or [1] * len(r["input_ids"]), dtype=torch.long)[: ids.numel()]
            if mask.numel() != ids.numel():
                raise ValueError(f"row {i}: loss_mask and input_ids differ in length")
            packed = pack_loss_mask(mask)
        out.append({"input_ids": ids, "packed_loss_mask": packed, "data_id": row_identity(r, i)})
    return out


def row_identity(row: dict, index: int) -> str:
    """A document's identity in ledgers, feature stores and seeds: the row's own ``data_id`` / ``id`` when it has one, else
    its place in the file."""
    for key in ("data_id", "id"):
        if row.get(key) not in (None, ""):
            return str(row[key])
    return str(index)


def preprocessing_identity(path: str, args: Mapping[str, Any]) -> str:
    keys = ("tokenizer_path", "target_model_path", "chat_template", "max_seq_length", "last_turn_loss_only", "renderer")
    body = {"file": _file_digest(path), "parser_version": PARSER_VERSION, **{k: args.get(k) for k in keys}}
    return hashlib.sha256(json.dumps(body, sort_keys=True, default=str).encode()).hexdigest()


def load_tokenizer(args: Mapping[str, Any]):
    path = args.get("tokenizer_path") or args.get("target_model_path")
    if not path:
        raise ValueError("conversation datasets need dataset.tokenizer_path or model.target_model_path")
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(path, local_files_only=True, trust_remote_code=bool(args.get("trust_remote_code", False)))


def load_training_samples(path: str, args: Mapping[str, Any], tokenizer=None, report: Optional[dict] = None) -> List[dict]:
    if not os.path.isfile(path):
        raise FileNotFoundError(f"training data not found: {path}")
    max_length = int(args["max_seq_length"])
    rows = read_rows(path)
    if is_pretokenized(rows):
        samples = _from_pretokenized(rows, max_length)
        if len({s["data_id"] for s in samples}) != len(samples):
            raise ValueError(f"{path}: two documents share one id; ids (data_id / id) must be unique")
        if report is not None:
            report.update({"seen": len(rows), "admitted": len(samples), "pretokenized": True})
        return samples
    cache_dir = args.get("cache_dir")
    cache_file = None
    if cache_dir:
        cache_file = os.path.join(cache_dir, "processed_dataset", preprocessing_identity(path, args) + ".pt")
        if os.path.isfile(cache_file):
            cached = torch.load(cache_file, weights_only=True)
            if report is not None:
                report.update({**cached["report"], "cache": "hit"})
            return cached["samples"]
    tokenizer = tokenizer or load_tokenizer(args)
    stats: Dict[str, Any] = {}
    if args.get("renderer"):
        from aspec_b200.data.renderers import RENDERER_REGISTRY
        renderer = RENDERER_REGISTRY.create(args["renderer"], tokenizer)
        samples = []
        for index, r in enumerate(rows):
            ids, mask = renderer.render(r.get("messages") or r.get("conversations"), tools=r.get("tools"),
                                        max_seq_length=max_length, last_turn_only=bool(args.get("last_turn_loss_only", False)))
            if int(mask.sum()):
                samples.append({"input_ids": ids, "packed_loss_mask": pack_loss_mask(mask), "source_index": index})
        stats = {"seen": len(rows), "admitted": len(samples), "renderer": args["renderer"]}
    else:
        parser = create_parser(tokenizer, TEMPLATE_REGISTRY.get(args.get("chat_template") or "qwen"))
        samples = preprocess_conversations(parser, (r.get("conversations") or r.get("messages") or [] for r in rows), max_length,
                                           args.get("last_turn_loss_only"), stats)
    for s in samples:                       # every document is named after its source row
        idx = int(s.pop("source_index"))
        s["data_id"] = row_identity(rows[idx], idx)
    if len({s["data_id"] for s in samples}) != len(samples):
        raise ValueError(f"{path}: two documents share one id; ids (data_id / id) must be unique")
    if cache_file:
        os.makedirs(os.path.dirname(cache_file), exist_ok=True)
        tmp = cache_file + ".tmp"
        torch.save({"samples": samples, "report": stats}, tmp)
        os.replace(tmp, cache_file)
    if report is not None:
        report.update({**stats, "cache": "miss" if cache_file else "off"})
    return samples
