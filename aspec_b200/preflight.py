"""Node preflight: what must hold before any actor is started.

Read-only checks of this node (the framework launches on one node): enough GPUs of one kind for the planned Target
and Draft pools, peer access between every pair that will exchange memory, memory headroom per GPU for the planned
estimate, shared-memory and run-directory headroom, the native libraries built for this source tree, a free rendezvous
port, and the NCCL settings that matter here (reference: aspec/ray/cluster_preflight.py:885-1277 - its per-node
probes and pairwise NVLink / RDMA checks, reduced to the single-node subset; nothing is changed on the machine).

The report's ``state`` is ``validated`` (all checks passed), ``failed`` (``problems`` lists why) or ``skipped`` (no GPU:
CPU runs need none of this).  ``train_entry`` refuses to start actors on ``failed``.
"""
from __future__ import annotations

import os
import shutil
import socket
from typing import Dict, List


def _port_free(port: int) -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        try:
            s.bind(("127.0.0.1", port))
            return True
        except OSError:
            return False


def run_cluster_preflight(flat: Dict) -> dict:
    checks: List[dict] = []

    def check(name: str, ok: bool, detail=None) -> None:
        checks.append({"name": name, "ok": bool(ok), "detail": detail})

    try:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:                                   # noqa: BLE001
        n = 0
    native = flat.get("inference_engine_type") == "native"
    targets = int(flat.get("inference_num_gpus") or 0) if native else 0
    # colocated roles share GPUs: the larger role sets the requirement
    need = max(int(flat["world_size"]), targets) if flat.get("colocate") else int(flat["world_size"]) + targets
    out = {"mode": flat.get("cluster_mode", "single_node"), "host": socket.gethostname(), "gpu_count": n,
           "visible_gpus": n, "required_gpus": need, "checks": checks}
    if n == 0 or flat.get("force_cpu"):
        out.update(state="skipped", ok=True, problems=[])
        return out
    import torch
    names = [torch.cuda.get_device_name(i) for i in range(n)]
    check("gpu_count", n >= need, {"visible": n, "required": need})
    check("homogeneous_gpus", len(set(names)) == 1, sorted(set(names)))
    caps = {torch.cuda.get_device_capability(i) for i in range(n)}
    check("compute_capability_10_x", all(c[0] == 10 for c in caps), sorted(caps))
    used = range(min(n, need))
    blocked = [(i, j) for i in used for j in used if i != j and not torch.cuda.can_device_access_peer(i, j)]
    check("peer_access", not blocked, blocked[:8])
    # memory: the plan's per-rank estimate must fit what is free now (other jobs may share the node)
    want = int((flat.get("memory_estimate_bytes") or 0))
    free = []
    for i in used:
        f, t = torch.cuda.mem_get_info(i)
        free.append({"gpu": i, "free_bytes": f, "total_bytes": t})
    check("gpu_memory_headroom", all(x["free_bytes"] > max(want, 1 << 30) for x in free), free)
    shm = shutil.disk_usage("/dev/shm") if os.path.isdir("/dev/shm") else None
    if shm:
        check("shared_memory_free_bytes", shm.free > (1 << 28), shm.free)
    run_dir = str(flat.get("output_dir") or ".")
    probe = run_dir if os.path.isdir(run_dir) else os.path.dirname(os.path.abspath(run_dir)) or "."
    try:
        check("run_directory_free_bytes", shutil.disk_usage(probe).free > (1 << 30), shutil.disk_usage(probe).free)
    except OSError as exc:
        check("run_directory_free_bytes", False, str(exc))
    from aspec_b200 import _native
    check("kernel_library_built", _native.kernels_available(), str(_native._KERNEL_LIB))
    stale = _native._stale(_native._KERNEL_LIB, sorted(_native._CSRC.glob("*.cu")) + sorted(_native._CSRC.glob("*.cuh"))
                           + sorted(_native._CSRC.glob("*.h"))) if _native.kernels_available() else True
    check("kernel_library_matches_sources", not stale, "run `python -m aspec_b200.build`" if stale else None)
    port = int(flat.get("master_port") or 0)
    if port:
        check("rendezvous_port_free", _port_free(port), port)
    # settings that change how collectives behave on this node; reported, never changed
    out["nccl_environment"] = {k: v for k, v in os.environ.items() if k.startswith("NCCL_")}
    problems = [c["name"] for c in checks if not c["ok"]]
    out.update(state="validated" if not problems else "failed", ok=not problems, problems=problems)
    return out
