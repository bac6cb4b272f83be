"""``doctor``: inspect the environment a run depends on - interpreter, torch / CUDA versions, compiler, the built
native libraries and their identity, and (with ``--gpu``) the visible GPUs and their peer paths
(reference: aspec/commands/doctor.py:30-200, which audits its pinned serving-engine dependency lane instead)."""
from __future__ import annotations

import argparse
import json
import os
import platform
import shutil
import subprocess
import sys


def inspect_environment(gpu: bool = False) -> dict:
    result = {"python": sys.executable, "python_version": platform.python_version(), "platform": platform.platform(),
              "gpu_requested": gpu, "checks": [], "errors": []}

    def check(name, ok, detail=""):
        result["checks"].append({"name": name, "ok": bool(ok), "detail": str(detail)})
        if not ok:
            result["errors"].append(f"{name}: {detail}")

    check("python>=3.10", sys.version_info[:2] >= (3, 10), platform.python_version())
    check("linux", sys.platform == "linux", sys.platform)
    try:
        import torch
        check("torch", True, torch.__version__)
        check("torch.distributed nccl+gloo", torch.distributed.is_nccl_available() and torch.distributed.is_gloo_available(), "")
    except Exception as exc:                                     # noqa: BLE001
        check("torch", False, exc)
        return result
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if os.path.exists(nvcc):
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.strip().splitlines()
        check("nvcc", True, out[-2] if len(out) > 1 else out)
    else:
        check("nvcc", False, "not found: the sm_100a kernels cannot be rebuilt")
    from aspec_b200 import _native
    lib_dir = os.path.join(os.path.dirname(os.path.abspath(_native.__file__)), "lib")
    for lib in ("libaspec_b200_kernels.so", "libaspec_b200_runtime.so"):
        path = os.path.join(lib_dir, lib)
        check(lib, os.path.isfile(path), path if os.path.isfile(path) else "missing: run `aspec-b200 build`")
    try:
        from aspec_b200.runtime_identity import runtime_identity
        result["runtime_identity"] = runtime_identity()["sha256"]
    except Exception as exc:                                     # noqa: BLE001
        check("runtime identity", False, exc)
    try:
        _native.runtime()
        check("runtime library loads", True)
    except Exception as exc:                                     # noqa: BLE001
        check("runtime library loads", False, exc)
    if gpu:
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        check("cuda available", n > 0, f"{n} device(s)")
        gpus = []
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "memory_gib": round(p.total_memory / 2 ** 30, 1),
                         "sms": p.multi_processor_count})
            check(f"gpu{i} is sm_100", (p.major, p.minor) == (10, 0), f"{p.name} sm_{p.major}{p.minor}")
        result["gpus"] = gpus
        if n > 1:
            result["peer_access"] = [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)] for i in range(n)]
            check("all GPU pairs have a peer path", all(all(r) for r in result["peer_access"]), "")
        if n:
            try:
                _native.kernels()
                check("kernel library loads", True)
            except Exception as exc:                             # noqa: BLE001
                check("kernel library loads", False, exc)
    return result


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 doctor", description=__doc__)
    ap.add_argument("--gpu", action="store_true", help="also inspect the visible GPUs (reads settings, changes none)")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    res = inspect_environment(a.gpu)
    if a.json:
        print(json.dumps(res, indent=2))
    else:
        for c in res["checks"]:
            print(("ok   " if c["ok"] else "FAIL ") + c["name"] + (f"  ({c['detail']})" if c["detail"] else ""))
        print("environment is ready" if not res["errors"] else f"{len(res['errors'])} problem(s) found")
    return 0 if not res["errors"] else 1


if __name__ == "__main__":
    sys.exit(main())
