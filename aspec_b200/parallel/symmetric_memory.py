"""Device buffers that several processes of one node map: the substrate of every peer-memory kernel.

``SymmetricBuffer.allocate`` makes one ``cudaMalloc`` allocation in the owner process and wraps it as a
``torch.uint8`` tensor; ``export()`` yields plain data (the 64-byte CUDA IPC handle) that can be relayed by
any process; ``SymmetricBuffer.open`` maps it in another process *with the accessing GPU current* and
presents it as a tensor of that GPU, so both torch ops and the framework's kernels treat peer HBM like
local memory (loads and stores travel over NVLink 5 through the NVSwitch).  On CPU (tests) the buffer is
ordinary shared memory.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from aspec_b200 import _native


class _RawCudaMemory:
    """Adapter that exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}
        self._owner = owner


class SymmetricBuffer:
    def __init__(self, tensor: torch.Tensor, ptr: Optional[int], owned: bool, imported: bool):
        self.tensor, self._ptr, self._owned, self._imported = tensor, ptr, owned, imported

    # -- owner ------------------------------------------------------------------------------------
    @classmethod
    def allocate(cls, nbytes: int, device) -> "SymmetricBuffer":
        device = torch.device(device)
        if device.type != "cuda":
            return cls(torch.zeros(nbytes, dtype=torch.uint8).share_memory_(), None, False, False)
        nbytes = -(-nbytes // 256) * 256
        with torch.cuda.device(device):
            torch.cuda.init()
            ptr = C.c_void_p()
            rc = _native.kernels().ab_symm_alloc(C.c_ulonglong(nbytes), C.byref(ptr))
            if rc != 0:
                raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed (code {rc})")
            t = torch.as_tensor(_RawCudaMemory(ptr.value, nbytes, None), device=device)
        return cls(t, ptr.value, True, False)

    def export(self) -> dict:
        if self._ptr is None:
            return {"kind": "cpu", "tensor": self.tensor}
        handle = (C.c_ubyte * 64)()
        rc = _native.kernels().ab_ipc_export(C.c_void_p(self._ptr), handle)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed (code {rc})")
        return {"kind": "cuda_ipc", "handle": bytes(handle), "nbytes": self.tensor.numel(),
                "device": self.tensor.device.index}

    # -- importer ---------------------------------------------------------------------------------
    @classmethod
    def open(cls, meta: dict, accessing_device=None) -> "SymmetricBuffer":
        if meta["kind"] == "cpu":
            return cls(meta["tensor"], None, False, False)
        dev = torch.device("cuda", torch.cuda.current_device()) if accessing_device is None else torch.device(accessing_device)
        with torch.cuda.device(dev):
            torch.cuda.init()
            torch.zeros(1, device=dev)       # make sure the primary context exists
            ptr = C.c_void_p()
            rc = _native.kernels().ab_ipc_import((C.c_ubyte * 64).from_buffer_copy(meta["handle"]), int(dev.index),
                                                 C.byref(ptr))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle failed (code {rc}); is peer access available between GPU "
                                   f"{dev.index} and GPU {meta['device']}?")
            t = torch.as_tensor(_RawCudaMemory(ptr.value, meta["nbytes"], None), device=dev)
        return cls(t, ptr.value, False, True)

    def close(self) -> None:
        if self._ptr is None:
            return
        lib = _native.kernels()
        if self._imported:
            lib.ab_ipc_close(C.c_void_p(self._ptr))
        elif self._owned:
            lib.ab_symm_free(C.c_void_p(self._ptr))
        self._ptr = None
