"""Guard bands around device allocations: a memory checker for kernel tests that needs no external tool.

Inside ``guard_allocations()`` every CUDA tensor made by ``torch.empty`` / ``zeros`` / ``ones`` / ``full`` /
``empty_like`` / ``zeros_like`` / ``ones_like`` (which is how the kernel wrappers in ``aspec_b200.ops`` allocate their outputs and
scratch) is carved out of a larger allocation with ``pad_bytes`` of a known byte pattern before and after it.  On exit
(or ``check()``) every band is compared with the pattern; a kernel that stored outside a buffer it was given - the
class of bug a bounds-checking build or a sanitizer would report - fails the block with the allocation's shape and the
offset of the first damaged byte.  Reads out of bounds are not seen; numerics tests against fp32 statements cover
those.  Meant for tests: allocations inside the block cost an extra fill and are kept alive until the block ends.
"""
from __future__ import annotations

import contextlib
import math
from typing import List, Tuple

import torch

PATTERN = 0xA5
_MAKERS = ("empty", "zeros", "ones", "full")
_LIKES = ("empty_like", "zeros_like", "ones_like")


class CanaryError(AssertionError):
    pass


class _Guard:
    def __init__(self, pad_bytes: int):
        self.pad = -(-int(pad_bytes) // 256) * 256          # keeps the inner tensor 256-byte aligned
        self.live: List[Tuple[torch.Tensor, int, tuple, torch.dtype]] = []

    def carve(self, shape, dtype, device, fill=None) -> torch.Tensor:
        shape = tuple(int(x) for x in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        nbytes = math.prod(shape) * torch.empty(0, dtype=dtype).element_size()
        inner = -(-nbytes // 256) * 256
        raw = _REAL["empty"](self.pad * 2 + inner, dtype=torch.uint8, device=device)
        raw.fill_(PATTERN)
        self.live.append((raw, nbytes, shape, dtype))
        view = raw[self.pad:self.pad + nbytes].view(dtype).view(shape)
        if fill is not None:
            view.fill_(fill)
        return view

    def check(self) -> None:
        for raw, nbytes, shape, dtype in self.live:
            for name, band, base in (("before", raw[: self.pad], -self.pad), ("after", raw[self.pad + nbytes:], nbytes)):
                bad = (band != PATTERN).nonzero()
                if bad.numel():
                    at = int(bad[0])
                    raise CanaryError(f"write outside a {dtype} buffer of shape {shape}: {int(bad.numel())} damaged guard bytes "
                                      f"{name} it, first at byte offset {base + at} relative to the buffer")


_REAL = {name: getattr(torch, name) for name in _MAKERS + _LIKES}


def _is_cuda(device) -> bool:
    return device is not None and torch.device(device).type == "cuda"


@contextlib.contextmanager
def guard_allocations(pad_bytes: int = 4096):
    guard = _Guard(pad_bytes)

    def maker(name):
        real = _REAL[name]

        def make(*size, **kw):
            device = kw.get("device")
            if not _is_cuda(device) or kw.get("out") is not None or kw.get("pin_memory") or kw.get("requires_grad"):
                return real(*size, **kw)
            fill = {"empty": None, "zeros": 0, "ones": 1}.get(name)
            if name == "full":
                *size, fill = size if len(size) == 2 else (size[0], kw.pop("fill_value"))
                size = size[0] if len(size) == 1 else size
                return guard.carve(size, kw.get("dtype") or (torch.get_default_dtype() if isinstance(fill, float) else torch.int64),
                                   device, fill)
            shape = size[0] if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)) else size
            return guard.carve(shape, kw.get("dtype") or torch.get_default_dtype(), device, fill)
        return make

    def like(name):
        real = _REAL[name]

        def make(t, **kw):
            device = kw.get("device", t.device)
            if not _is_cuda(device) or kw.get("requires_grad") or (not t.is_contiguous() and "memory_format" not in kw):
                return real(t, **kw)
            return guard.carve(t.shape, kw.get("dtype") or t.dtype, device, {"empty_like": None, "zeros_like": 0, "ones_like": 1}[name])
        return make

    for name in _MAKERS:
        setattr(torch, name, maker(name))
    for name in _LIKES:
        setattr(torch, name, like(name))
    try:
        yield guard
        guard.check()
    finally:
        for name, fn in _REAL.items():
            setattr(torch, name, fn)
