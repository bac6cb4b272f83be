"""Runtime identity: a SHA-256 over a bounded, ordered list of files that define the numerical behaviour of a run
(kernel sources, the built libraries, the package version).  Stored in plans, evidence, offline bindings and
checkpoints so that a resume or a replay under different kernels is detected
(reference: aspec/runtime_identity.py:28-119, which hashes the serving engine's files for the same purpose)."""
from __future__ import annotations

import hashlib
import os
from typing import Dict, Iterable, List, Optional

_PACKAGE = os.path.dirname(os.path.abspath(__file__))
IDENTITY_FILES = ("csrc/common.cuh", "csrc/gemm_sm100.cu", "csrc/attention_fwd_sm100.cu", "csrc/attention_bwd_sm100.cu",
                  "csrc/elementwise_sm100.cu", "csrc/comm_sm100.cu", "csrc/runtime/slot_ring.cpp",
                  "csrc/runtime/work_ledger.cpp", "csrc/runtime/packer.cpp")
MAX_FILE_BYTES = 16 << 20


def file_sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def runtime_identity(files: Optional[Iterable[str]] = None, root: str = _PACKAGE) -> Dict:
    entries: List[Dict] = []
    outer = hashlib.sha256()
    for rel in (files if files is not None else IDENTITY_FILES):
        path = os.path.join(root, rel)
        if not os.path.isfile(path):
            raise FileNotFoundError(f"runtime identity file missing: {rel}")
        if os.path.getsize(path) > MAX_FILE_BYTES:
            raise ValueError(f"runtime identity file too large: {rel}")
        digest = file_sha256(path)
        entries.append({"file": rel, "sha256": digest})
        outer.update(rel.encode() + b"\0" + digest.encode() + b"\n")
    from aspec_b200 import __version__
    outer.update(("version\0" + __version__).encode())
    return {"schema": "aspec.runtime-identity/v1", "version": __version__, "files": entries, "sha256": outer.hexdigest()}


def verify_runtime_identity(expected: Dict, root: str = _PACKAGE) -> None:
    actual = runtime_identity([e["file"] for e in expected["files"]], root)
    if actual["sha256"] != expected["sha256"]:
        changed = [a["file"] for a, e in zip(actual["files"], expected["files"]) if a["sha256"] != e["sha256"]]
        raise ValueError(f"runtime identity mismatch; changed files: {changed or ['package version']}")
