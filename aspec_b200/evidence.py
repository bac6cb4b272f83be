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


class EvidenceError(RuntimeError):
    """An observation that contradicts the plan (or itself).  Evidence never records a claim it cannot stand behind."""


# capability -> what must have been observed for the capability to count as exercised by this run
ACTIVATION_RULES = {
    "feature_transport": "an optimizer step consumed Target features whose contract id equals the planned one",
    "attention": "rank 0 launched the planned attention implementation at least once",
    "gemm": "rank 0 launched the planned GEMM implementation at least once",
    "data_parallel": "more than one Draft rank completed an optimizer step",
    "context_parallel": "a context-parallel group completed an optimizer step",
    "expert_parallel": "an expert-parallel group completed an optimizer step",
    "vocab_parallel": "a vocabulary-parallel group completed an optimizer step",
    "work_ledger": "the ledger validated: every committed work id was registered, dispatched and released exactly once",
}


class RunEvidenceRecorder:
    """Typed observations of one run, each checked against the plan before it is written
    (reference: aspec/evidence.py:271-1624; sections restated for this framework's process model).

    Sections: ``dataset_admission`` -> ``actor_initialization`` -> ``cluster_preflight`` -> ``training`` -> ``cleanup``;
    ``capabilities_planned`` (from the plan), ``capabilities_observed`` (launch counts) and ``capabilities_activated``
    (planned capabilities whose activation rule was met, with the observation that met it)."""

    PHASES = ("created", "dataset_loaded", "actors_initialized", "training", "completed", "failed")

    def __init__(self, plan, output_dir: str):
        self.path = os.path.join(output_dir, "evidence.json")
        self._plan = plan
        self.doc: Dict[str, Any] = {
            "schema_version": SCHEMA, "plan_id": plan.plan_id, "framework_version": __version__,
            "package_sha256": package_hash(), "host": socket.gethostname(), "platform": platform.platform(),
            "started_at": time.time(), "accelerators": accelerator_inventory(), "phase": "created",
            "capabilities_planned": [c.__dict__ for c in plan.capabilities], "capabilities_activated": {},
            "sections": {}, "state": "running"}
        self._write()

    # -- plumbing -------------------------------------------------------------------------------------------
    def _write(self) -> None:
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.doc, f, indent=2, sort_keys=True, default=str)
        os.replace(tmp, self.path)

    def _policy(self) -> dict:
        return dict(getattr(self._plan, "policy", None) or {})

    def _planned(self, subsystem: str):
        for c in self._plan.capabilities:
            if c.subsystem == subsystem:
                return c
        return None

    @staticmethod
    def _choice(decision):
        return getattr(decision, "choice", getattr(decision, "planned", None))

    def _activate(self, subsystem: str, observation: dict) -> None:
        if self._planned(subsystem) is None:
            return
        self.doc["capabilities_activated"][subsystem] = {"rule": ACTIVATION_RULES.get(subsystem, "observed"),
                                                          "planned": self._choice(self._planned(subsystem)), **observation}

    def record(self, section: str, payload: Any) -> None:
        """Free-form section (kept for callers with observations of their own)."""
        self.doc["sections"][section] = payload
        self._write()

    # -- typed sections ----------------------------------------------------------------------------------------
    def record_dataset_admission(self, *, dataset_size: int, eval_dataset_size: int = 0, admission: Optional[dict] = None) -> None:
        """Source-to-runtime accounting, written before the expensive actor start-up.

        ``admission``: ``{"source_rows", "admitted", "rejected": {reason: count}, "fingerprint"}``.  Every source row is
        either admitted or rejected for a named reason; the admitted count is the dataset the controller will serve."""
        adm = dict(admission or {})
        rejected = {str(k): int(v) for k, v in (adm.get("rejected") or {}).items()}
        if any(v < 0 for v in rejected.values()) or dataset_size < 0 or eval_dataset_size < 0:
            raise EvidenceError("dataset admission counts must be non-negative")
        admitted = int(adm.get("admitted", dataset_size))
        if admitted != int(dataset_size):
            raise EvidenceError(f"admitted rows ({admitted}) differ from the dataset the controller serves ({dataset_size})")
        source = adm.get("source_rows")
        if source is not None and int(source) != admitted + sum(rejected.values()):
            raise EvidenceError(f"dataset admission does not add up: {source} source rows != {admitted} admitted + "
                                f"{sum(rejected.values())} rejected")
        self.doc["sections"]["dataset_admission"] = {
            "dataset_size": int(dataset_size), "eval_dataset_size": int(eval_dataset_size), "admitted": admitted,
            "source_rows": int(source) if source is not None else admitted, "rejected": rejected,
            "fingerprint": adm.get("fingerprint")}
        self.doc["phase"] = "dataset_loaded"
        self._write()

    def record_actor_initialization(self, *, training_actors: list, inference_engines: list) -> None:
        """Who runs where.  ``training_actors`` / ``inference_engines``: one ``{"name", "device", "pid"}`` per process.
        The counts must be the plan's, and no two processes may own the same GPU."""
        pol = self._policy()
        want_d, want_t = pol.get("draft_gpus"), pol.get("target_gpus")
        if want_d is not None and len(training_actors) != int(want_d):
            raise EvidenceError(f"initialised {len(training_actors)} Draft trainers, the plan has {want_d}")
        if want_t and len(inference_engines) != int(want_t):
            raise EvidenceError(f"initialised {len(inference_engines)} Target engines, the plan has {want_t}")
        gpus = [a.get("device") for a in list(training_actors) + list(inference_engines)
                if str(a.get("device", "")).startswith("cuda")]
        if len(gpus) != len(set(gpus)):
            raise EvidenceError(f"two processes were placed on one GPU: {sorted(gpus)}")
        self.doc["sections"]["actor_initialization"] = {
            "training_actor_count": len(training_actors), "inference_engine_count": len(inference_engines),
            "training_actors": list(training_actors), "inference_engines": list(inference_engines)}
        self.doc["phase"] = "actors_initialized"
        self._write()

    def record_cluster_preflight(self, report: dict) -> None:
        """The node check that ran before any actor: it must have passed, and it must cover the GPUs the plan uses."""
        if report.get("state") not in ("validated", "skipped"):
            raise EvidenceError(f"cluster preflight did not validate: {report.get('state')!r} {report.get('problems')}")
        pol = self._policy()
        roles = (int(pol.get("draft_gpus") or 0), int(pol.get("target_gpus") or 0))
        need = max(roles) if pol.get("colocate") else sum(roles)          # colocated roles share GPUs
        have = report.get("gpu_count")
        if report.get("state") == "validated" and have is not None and need and int(have) < need:
            raise EvidenceError(f"preflight saw {have} GPUs, the plan needs {need}")
        self.doc["sections"]["cluster_preflight"] = dict(report)
        self._write()

    def record_training(self, summary: dict) -> None:
        """The loop's summary; activates the capabilities whose rule the observations meet."""
        s = {k: v for k, v in dict(summary).items() if k not in ("history", "cleanup")}
        steps = int(s.get("optimizer_steps_observed", s.get("completed_steps", s.get("steps", 0))) or 0)
        ledger = s.get("ledger") or {}
        if steps > 0 and ledger and not ledger.get("validated", False):
            raise EvidenceError(f"the work ledger did not validate: {ledger}")
        self.doc["sections"]["training"] = s
        self.doc["phase"] = "training"
        pol = self._policy()
        if steps > 0:
            contract = s.get("feature_contract") or {}
            if not contract or contract.get("state") == "validated":
                self._activate("feature_transport", {"optimizer_steps_observed": steps,
                                                     "feature_contract_id": contract.get("contract_id")})
            if ledger.get("validated"):
                self.doc["capabilities_activated"]["work_ledger"] = {"rule": ACTIVATION_RULES["work_ledger"],
                                                                       "committed": ledger.get("committed")}
            if int(pol.get("draft_gpus") or 1) > 1:
                self._activate("data_parallel", {"optimizer_steps_observed": steps, "draft_gpus": pol.get("draft_gpus")})
            for key, subsystem in (("context_parallel", "context_parallel"), ("expert_parallel", "expert_parallel"),
                                   ("vocab_parallel", "vocab_parallel")):
                if int(pol.get(key) or 1) > 1:
                    self._activate(subsystem, {"optimizer_steps_observed": steps, "degree": pol.get(key)})
        observed = s.get("capabilities_observed") or self.doc.get("capabilities_observed") or {}
        for subsystem in ("attention", "gemm"):
            planned = self._planned(subsystem)
            seen = observed.get(subsystem)
            if planned is None or not seen:
                continue
            choice = self._choice(planned)
            launches = seen.get(choice, 0) if isinstance(seen, dict) else int(seen == choice)
            if launches:
                self._activate(subsystem, {"launches": launches})
        self._write()

    def record_cleanup(self, cleanup: dict) -> None:
        """How the processes ended: engines (accessors of the rings) must be observed gone before trainers (owners)."""
        c = dict(cleanup)
        order = c.get("order") or []
        if "trainers" in order and "engines" in order and order.index("trainers") < order.index("engines"):
            raise EvidenceError("trainers were released before the engines that store into their memory")
        self.doc["sections"]["cleanup"] = c
        self._write()

    def observe_capability(self, subsystem: str, observed: Any) -> None:
        """What really ran for ``subsystem``: an implementation name, or ``{implementation: launches}``."""
        self.doc.setdefault("capabilities_observed", {})[subsystem] = observed
        self._write()

    def complete(self, summary: Optional[dict] = None) -> None:
        if summary and "training" not in self.doc["sections"] and not summary.get("preflight_only"):
            self.record_training(summary)
        self.doc.update(state="completed", phase="completed", finished_at=time.time(), training_summary=summary or {})
        self._write()

    def fail(self, exc: BaseException) -> None:
        self.doc.update(state="failed", phase="failed", finished_at=time.time(),
                        failure={"type": type(exc).__name__, "message": str(exc),
                                 "traceback": "".join(traceback.format_exception(type(exc), exc, exc.__traceback__))[-8000:]})
        self._write()
