"""Node preflight: enough GPUs of one kind, peer access between every pair, shared-memory headroom
(reference: aspec/ray/cluster_preflight.py:885-1277, single-node subset; read-only queries)."""
from __future__ import annotations

import shutil
from typing import Dict


def run_cluster_preflight(flat: Dict) -> dict:
    out = {"mode": flat.get("cluster_mode", "single_node"), "checks": [], "ok": True}
    try:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:                                   # noqa: BLE001
        n = 0
    need = int(flat["world_size"]) + (int(flat["inference_num_gpus"]) if flat["inference_engine_type"] == "native" else 0)
    out["visible_gpus"], out["required_gpus"] = n, need
    if n:
        import torch
        names = {torch.cuda.get_device_name(i) for i in range(n)}
        out["checks"].append({"name": "homogeneous_gpus", "ok": len(names) == 1, "detail": sorted(names)})
        pairs_ok = all(torch.cuda.can_device_access_peer(i, j) for i in range(min(n, need)) for j in range(min(n, need)) if i != j)
        out["checks"].append({"name": "peer_access", "ok": pairs_ok})
        out["checks"].append({"name": "gpu_count", "ok": n >= need})
    shm = shutil.disk_usage("/dev/shm") if shutil.os.path.isdir("/dev/shm") else None
    if shm:
        out["checks"].append({"name": "shared_memory_free_bytes", "ok": shm.free > (1 << 28), "detail": shm.free})
    out["ok"] = all(c["ok"] for c in out["checks"]) if n else True
    return out
