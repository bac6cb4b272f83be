"""``evidence.json``: what actually happened, bound to the plan that was promised.

Written atomically after every recorded section; holds plan id, source and package hashes, accelerator
inventory, capability activation, dataset admission, placement, the training summary with the committed
work and throughput window, and how the run ended (reference: aspec/evidence.py:271-1624).
"""
from __future__ import annotations

import hashlib
import json
import os
import platform
import socket
import time
import traceback
from typing import Any, Dict, Optional

from aspec_b200 import __version__

SCHEMA = "aspec.run-evidence/v1"


def package_hash() -> str:
    root = os.path.dirname(os.path.abspath(__file__))
    h = hashlib.sha256()
    for base, _dirs, files in sorted(os.walk(root)):
        if "__pycache__" in base or os.sep + "lib" in base:
            continue
        for name in sorted(files):
            if name.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".json")):
                p = os.path.join(base, name)
                h.update(os.path.relpath(p, root).encode())
                h.update(open(p, "rb").read())
    return h.hexdigest()


def accelerator_inventory() -> dict:
    try:
        import torch
        if not torch.cuda.is_available():
            return {"cuda": False, "devices": []}
        devs = []
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            devs.append({"index": i, "name": p.name, "capability": f"{p.major}.{p.minor}",
                         "memory_bytes": p.total_memory, "sms": p.multi_processor_count})
        return {"cuda": True, "devices": devs, "torch": torch.__version__, "cuda_runtime": torch.version.cuda}
    except Exception as exc:                         # noqa: BLE001
        return {"cuda": False, "error": str(exc)}


class RunEvidenceRecorder:
    def __init__(self, plan, output_dir: str):
        self.path = os.path.join(output_dir, "evidence.json")
        self.doc: Dict[str, Any] = {
            "schema_version": SCHEMA, "plan_id": plan.plan_id, "framework_version": __version__,
            "package_sha256": package_hash(), "host": socket.gethostname(), "platform": platform.platform(),
            "started_at": time.time(), "accelerators": accelerator_inventory(),
            "capabilities_planned": [c.__dict__ for c in plan.capabilities], "sections": {}, "state": "running"}
        self._write()

    def _write(self) -> None:
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.doc, f, indent=2, sort_keys=True, default=str)
        os.replace(tmp, self.path)

    def record(self, section: str, payload: Any) -> None:
        self.doc["sections"][section] = payload
        self._write()

    def observe_capability(self, subsystem: str, observed: Any) -> None:
        """What really ran for ``subsystem``: an implementation name, or ``{implementation: launches}``."""
        self.doc.setdefault("capabilities_observed", {})[subsystem] = observed
        self._write()

    def complete(self, summary: Optional[dict] = None) -> None:
        self.doc.update(state="completed", finished_at=time.time(), training_summary=summary or {})
        self._write()

    def fail(self, exc: BaseException) -> None:
        self.doc.update(state="failed", finished_at=time.time(),
                        failure={"type": type(exc).__name__, "message": str(exc),
                                 "traceback": "".join(traceback.format_exception(type(exc), exc, exc.__traceback__))[-8000:]})
        self._write()
