"""Offline feature dataset: ``dataset.json`` (schema version, Target binding, completeness), one append-only
``manifest.jsonl`` (split, data_id, file, seq_len, sha256) and self-describing ``samples/*.pt`` records
(reference: aspec/offline/dataset.py:43-318).

A dataset is bound to the Target that produced it (model identity + feature contract); a consumer with another
contract is refused.  Records are verified against their manifest hash on load.  Writers append a sample file
first and its manifest row second, so a crash leaves at most an orphan file, never a dangling row.
"""
from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path
from typing import Any, Dict, Iterator, List, Optional

import torch

from aspec_b200.feature_contract import FeatureContractRuntime

OFFLINE_SCHEMA_VERSION = "aspec.offline-features/v1"


def _sha256(path: Path) -> str:
    h = hashlib.sha256()
    with path.open("rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


class OfflineFeatureStore:
    def __init__(self, root, *, create: bool = False, binding: Optional[dict] = None,
                 last_hidden_states_prenorm: Optional[bool] = None, allow_incomplete: bool = False):
        self.root = Path(root).expanduser().resolve()
        if create and self.root.exists() and any(self.root.iterdir()):
            raise FileExistsError(f"Offline output must be a new or empty directory: {self.root}")
        if create and not binding:
            raise ValueError("Materialization requires a Target feature binding")
        meta = self.root / "dataset.json"
        if create:
            (self.root / "samples").mkdir(parents=True, exist_ok=True)
            meta.write_text(json.dumps({"version": OFFLINE_SCHEMA_VERSION, "binding": binding, "complete": False,
                                        "last_hidden_states_prenorm": last_hidden_states_prenorm}, indent=2) + "\n")
        if not meta.is_file():
            raise FileNotFoundError(f"Offline dataset not found: {meta}")
        self.metadata = json.loads(meta.read_text())
        if self.metadata.get("version") != OFFLINE_SCHEMA_VERSION:
            raise ValueError(f"Unsupported offline dataset version {self.metadata.get('version')!r}")
        if not (create or allow_incomplete) and not self.metadata.get("complete"):
            raise ValueError("Offline dataset is incomplete; finish materialization first")
        self.binding = self.metadata["binding"]
        self.contract = FeatureContractRuntime(self.binding["feature_contract"], role="consumer" if not create else "producer",
                                               participant="offline_dataset")
        self._rows: Dict[str, List[dict]] = {"train": [], "eval": []}
        self._by_id: Dict[str, dict] = {}
        manifest = self.root / "manifest.jsonl"
        if manifest.exists():
            for lineno, line in enumerate(manifest.read_text().splitlines(), 1):
                if not line.strip():
                    continue
                row = json.loads(line)
                split, data_id = row.get("split"), str(row.get("data_id"))
                if split not in self._rows:
                    raise ValueError(f"Invalid split in {manifest}:{lineno}")
                if data_id in self._by_id:
                    raise ValueError(f"Duplicate data_id {data_id!r} in {manifest}")
                path = (self.root / row["file"]).resolve()
                if self.root not in path.parents or not path.is_file():
                    raise FileNotFoundError(f"Offline sample not found: {path}")
                item = {k: row[k] for k in ("split", "file", "seq_len", "sha256")}
                item["data_id"] = data_id
                self._rows[split].append(item)
                self._by_id[data_id] = item

    # -- reading ------------------------------------------------------------------------------------------------
    def validate_consumer(self, contract_id: str) -> None:
        self.contract.validate_binding(contract_id)

    def rows(self, split: str = "train") -> List[dict]:
        return list(self._rows[split])

    def __len__(self) -> int:
        return len(self._by_id)

    def load(self, data_id, verify: bool = True) -> Dict[str, Any]:
        row = self._by_id[str(data_id)]
        path = self.root / row["file"]
        if verify and _sha256(path) != row["sha256"]:
            raise ValueError(f"Offline sample {path} does not match its manifest hash")
        rec = torch.load(path, map_location="cpu", weights_only=True)
        if int(rec["input_ids"].shape[-1]) != int(row["seq_len"]):
            raise ValueError(f"Offline sample {path} has a different length than its manifest row")
        return rec

    def samples(self, split: str = "train") -> Iterator[dict]:
        """Controller-side sample descriptors (ids and packed loss mask only; features stay on disk)."""
        from aspec_b200.data.utils import pack_loss_mask
        for row in self._rows[split]:
            rec = self.load(row["data_id"], verify=False)
            yield {"data_id": row["data_id"], "input_ids": rec["input_ids"].reshape(-1),
                   "packed_loss_mask": rec.get("packed_loss_mask") or pack_loss_mask(rec["loss_mask"].reshape(-1))}

    # -- writing ------------------------------------------------------------------------------------------------
    def append(self, split: str, data_id, record: Dict[str, Any]) -> dict:
        if split not in self._rows:
            raise ValueError(f"Invalid split {split!r}")
        data_id = str(data_id)
        if data_id in self._by_id:
            raise ValueError(f"Duplicate data_id {data_id!r}")
        payload = {k: v for k, v in record.items() if k in self.contract.contract["tensors"]}
        self.contract.validate_payload(payload)
        rel = f"samples/{split}-{len(self._rows[split]):08d}.pt"
        path = self.root / rel
        tmp = path.with_suffix(".pt.tmp")
        torch.save({k: (v.contiguous() if torch.is_tensor(v) else v) for k, v in record.items()}, tmp)
        os.replace(tmp, path)
        row = {"split": split, "data_id": data_id, "file": rel, "seq_len": int(record["input_ids"].shape[-1]),
               "sha256": _sha256(path)}
        with (self.root / "manifest.jsonl").open("a") as f:
            f.write(json.dumps(row) + "\n")
            f.flush()
            os.fsync(f.fileno())
        self._rows[split].append(row)
        self._by_id[data_id] = row
        return row

    def mark_complete(self) -> None:
        self.metadata["complete"] = True
        tmp = self.root / "dataset.json.tmp"
        tmp.write_text(json.dumps(self.metadata, indent=2) + "\n")
        os.replace(tmp, self.root / "dataset.json")
