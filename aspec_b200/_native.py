"""Builds and loads the in-tree native libraries.

Two shared objects live next to this file under ``lib/``:

* ``libaspec_b200_kernels.so`` - every hand-written sm_100a CUDA kernel
  (``csrc/*.cu``), compiled by ``nvcc -gencode arch=compute_100a,code=sm_100a``
  and exported through a plain C ABI that is called with raw device pointers
  and a stream handle;
* ``libaspec_b200_runtime.so`` - the host runtime in C++ (``csrc/runtime/*.cpp``):
  slot rings with generation leases, the work ledger, the row packer.

The kernels are called through ``ctypes`` so they depend on neither the torch
headers nor a particular torch ABI, and so that callers other than Python can
link the same symbols.  On a machine with a GPU a missing kernel library is an
error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_ROOT = Path(__file__).resolve().parent
_CSRC = _ROOT / "csrc"
_LIBDIR = _ROOT / "lib"
_KERNEL_LIB = _LIBDIR / "libaspec_b200_kernels.so"
_RUNTIME_LIB = _LIBDIR / "libaspec_b200_runtime.so"
_lock = threading.Lock()
_kernels = None
_runtime = None

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _stale(lib: Path, sources) -> bool:
    stamp = lib.with_suffix(".sha256")
    if not lib.exists() or not stamp.exists():
        return True
    return stamp.read_text().strip() != _digest(sources)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link one shared object."""
    sources = sorted(_CSRC.glob("*.cu"))
    headers = sorted(_CSRC.glob("*.cuh")) + sorted(_CSRC.glob("*.h"))
    if not force and not _stale(_KERNEL_LIB, sources + headers):
        return _KERNEL_LIB
    _LIBDIR.mkdir(exist_ok=True)
    objdir = _LIBDIR / "obj"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(_CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    cmd = [nvcc, "-shared", "-o", str(_KERNEL_LIB), *map(str, objs), "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    _KERNEL_LIB.with_suffix(".sha256").write_text(_digest(sources + headers))
    return _KERNEL_LIB


def build_runtime(force: bool = False) -> Path:
    """Compile the host runtime (``csrc/runtime/*.cpp``) with g++."""
    sources = sorted((_CSRC / "runtime").glob("*.cpp"))
    headers = sorted((_CSRC / "runtime").glob("*.h"))
    if not sources:
        return _RUNTIME_LIB
    if not force and not _stale(_RUNTIME_LIB, sources + headers):
        return _RUNTIME_LIB
    _LIBDIR.mkdir(exist_ok=True)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", str(_RUNTIME_LIB),
           *map(str, sources)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{res.stdout}\n{res.stderr}")
    _RUNTIME_LIB.with_suffix(".sha256").write_text(_digest(sources + headers))
    return _RUNTIME_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_runtime(force=force)


# GPU kernels launched by one call of each exported entry point (for launch accounting).
_LAUNCHES_PER_CALL = {"ab_attn_bwd": 3}
launch_count = 0


class _CountingLibrary:
    """Forwards to the ctypes library and counts kernel launches made through it."""

    def __init__(self, lib: ctypes.CDLL):
        self._lib = lib
        self._cache = {}

    def __getattr__(self, name: str):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._lib, name)
            weight = _LAUNCHES_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _w=weight):
                global launch_count
                launch_count += _w
                return _raw(*args)

            self._cache[name] = fn
        return fn


def kernels() -> "_CountingLibrary":
    """The CUDA kernel library.  Raises if it has not been built."""
    global _kernels
    with _lock:
        if _kernels is None:
            if not _KERNEL_LIB.exists():
                raise RuntimeError(
                    f"{_KERNEL_LIB} is missing: run `python -m aspec_b200.build` first")
            _kernels = _CountingLibrary(ctypes.CDLL(str(_KERNEL_LIB)))
        return _kernels


def runtime() -> ctypes.CDLL:
    """The C++ host runtime library; built on first use (g++ only, seconds)."""
    global _runtime
    with _lock:
        if _runtime is None:
            build_runtime()
            _runtime = ctypes.CDLL(str(_RUNTIME_LIB))
        return _runtime


def kernels_available() -> bool:
    return _KERNEL_LIB.exists()
