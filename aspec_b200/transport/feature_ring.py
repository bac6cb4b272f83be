"""Feature rings: Target -> Draft tensors move by stores into the consumer's own GPU memory.

Replaces the reference's Mooncake TransferEngine path (aspec/transfer/mooncake/p2p.py:684-1706,
aspec/inference/target_prefill.py:40-326).  The *consumer* (a Draft rank) owns a ring of fixed-size slots
in its HBM and exports it (CUDA IPC) to the Target ranks; the Target's captured-layer GEMM epilogues and
its final norm write ``hidden_states`` / ``last_hidden_states`` straight into the leased slot over
NVLink, so there is no source ring, no staging copy and no pull.  The lease protocol is the
generation-checked one of ``transport.slot_ring``; a descriptor names run, attempt, consumer, slot and
generation and a stale one is rejected before any byte is read.

Readiness: by default the producer synchronises its stream before it reports the descriptor (host
ordered).  With ``device_flags=True`` it instead publishes the generation into the slot's flag word
from the device and the consumer enqueues a bounded wait kernel, keeping both hosts out of the path.
Tensors inside a slot start on 256-byte boundaries.
"""
from __future__ import annotations

import base64
import ctypes as C
import json
from dataclasses import dataclass
from typing import Dict, Optional

import torch

KEY_PREFIX = "aspec-p2p-v3:"
ALIGN = 256


def _up(n: int, a: int = ALIGN) -> int:
    return -(-n // a) * a


@dataclass(frozen=True)
class SlotLayout:
    max_tokens: int
    num_layers: int
    hidden: int
    store_last_hidden: bool = True
    dtype: str = "bfloat16"

    @property
    def elem(self) -> int:
        return torch.empty(0, dtype=getattr(torch, self.dtype)).element_size()

    @property
    def offsets(self) -> Dict[str, int]:
        ids = 0
        hs = _up(ids + self.max_tokens * 8)
        last = _up(hs + self.max_tokens * self.num_layers * self.hidden * self.elem)
        end = _up(last + (self.max_tokens * self.hidden * self.elem if self.store_last_hidden else 0))
        return {"input_ids": ids, "hidden_states": hs, "last_hidden_states": last, "end": end}

    @property
    def slot_bytes(self) -> int:
        return self.offsets["end"]

    def to_dict(self) -> dict:
        return {"max_tokens": self.max_tokens, "num_layers": self.num_layers, "hidden": self.hidden,
                "store_last_hidden": self.store_last_hidden, "dtype": self.dtype}


def feature_bytes(n_tokens: int, num_layers: int, hidden: int, elem: int = 2, last: bool = True) -> int:
    """Payload of one sample (sizing rule of aspec/transfer/mooncake/helpers.py:36-116)."""
    return n_tokens * 8 + n_tokens * num_layers * hidden * elem + (n_tokens * hidden * elem if last else 0)


@dataclass(frozen=True)
class FeatureDescriptor:
    run_id: str
    attempt_id: str
    consumer: int
    slot: int
    generation: int
    n_tokens: int
    layer_ids: tuple
    hidden: int
    dtype: str = "bfloat16"
    view_start: int = 0            # context-parallel / layer sub-views of one slot
    view_end: Optional[int] = None

    def to_key(self) -> str:
        body = json.dumps(self.__dict__, sort_keys=True, separators=(",", ":"), default=list)
        return KEY_PREFIX + base64.urlsafe_b64encode(body.encode()).decode()

    @classmethod
    def from_key(cls, key: str) -> "FeatureDescriptor":
        if not key.startswith(KEY_PREFIX):
            raise ValueError("not a feature descriptor key")
        raw = json.loads(base64.urlsafe_b64decode(key[len(KEY_PREFIX):].encode()))
        raw["layer_ids"] = tuple(raw["layer_ids"])
        return cls(**raw)

    def tensor_shapes(self) -> dict:
        return {"input_ids": (self.n_tokens,), "hidden_states": (self.n_tokens, len(self.layer_ids) * self.hidden),
                "last_hidden_states": (self.n_tokens, self.hidden)}


def export_tensor(t: torch.Tensor) -> dict:
    """Plain-data handle of a tensor for ONE receiving process.

    CUDA: the IPC handle of the storage (``_share_cuda_``); being plain data it can be relayed by a third
    process (the driver), which ``torch.multiprocessing``'s own tensor pickling does not allow.  Call once
    per receiver: every export takes one reference that the receiver's import releases.
    CPU: the tensor itself, in shared memory.
    """
    if not t.is_cuda:
        return {"kind": "cpu", "tensor": t if t.is_shared() else t.share_memory_()}
    return {"kind": "cuda", "share": tuple(t.untyped_storage()._share_cuda_()), "dtype": str(t.dtype).split(".")[1],
            "shape": tuple(t.shape), "stride": tuple(t.stride()), "offset": t.storage_offset()}


def ensure_peer_access(local_device, peer_device) -> None:
    """Kernels on ``local_device`` are about to store into memory of ``peer_device``."""
    local, peer = torch.device(local_device), torch.device(peer_device)
    if local.type != "cuda" or peer.type != "cuda" or local.index == peer.index:
        return
    from aspec_b200 import _native
    rc = _native.kernels().ab_enable_peer_access(int(local.index), int(peer.index))
    if rc != 0:
        raise RuntimeError(f"GPU {local.index} cannot open peer access to GPU {peer.index} (code {rc})")


def import_tensor(meta: dict) -> torch.Tensor:
    if meta["kind"] == "cpu":
        return meta["tensor"]
    storage = torch.UntypedStorage._new_shared_cuda(*meta["share"])
    dtype = getattr(torch, meta["dtype"])
    out = torch.empty(0, dtype=dtype, device=storage.device)
    out.set_(storage, meta["offset"], meta["shape"], meta["stride"])
    return out


class _SlotViews:
    def __init__(self, buffer: torch.Tensor, flags: torch.Tensor, layout: SlotLayout, slots: int):
        self.buffer, self.flags, self.layout, self.slots = buffer, flags, layout, slots

    def views(self, slot: int, n_tokens: int) -> Dict[str, torch.Tensor]:
        lay = self.layout
        if not 0 <= slot < self.slots or not 0 < n_tokens <= lay.max_tokens:
            raise ValueError(f"slot {slot} / {n_tokens} tokens outside the ring")
        base = slot * lay.slot_bytes
        off = lay.offsets
        dt = getattr(torch, lay.dtype)
        raw = self.buffer
        ids = raw[base + off["input_ids"]: base + off["input_ids"] + n_tokens * 8].view(torch.int64)
        width = lay.num_layers * lay.hidden
        hs = raw[base + off["hidden_states"]: base + off["hidden_states"] + n_tokens * width * lay.elem] \
            .view(dt).view(n_tokens, width)
        out = {"input_ids": ids, "hidden_states": hs}
        if lay.store_last_hidden:
            out["last_hidden_states"] = raw[base + off["last_hidden_states"]:
                                            base + off["last_hidden_states"] + n_tokens * lay.hidden * lay.elem] \
                .view(dt).view(n_tokens, lay.hidden)
        return out


class FeatureRing(_SlotViews):
    """Consumer side: allocates the slots (and one flag word per slot) on its own device."""

    def __init__(self, slots: int, layout: SlotLayout, device, run_id: str = "run", attempt_id: str = "0",
                 consumer: int = 0):
        from aspec_b200.parallel.symmetric_memory import SymmetricBuffer
        device = torch.device(device)
        # one allocation: [slots * slot_bytes of payload][slots int64 flag words]
        payload = slots * layout.slot_bytes
        self._symm = SymmetricBuffer.allocate(payload + _up(slots * 8), device)
        raw = self._symm.tensor
        buffer = raw[:payload]
        flags = raw[payload:payload + slots * 8].view(torch.int64)
        super().__init__(buffer, flags, layout, slots)
        self.run_id, self.attempt_id, self.consumer = run_id, attempt_id, consumer
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def export(self) -> dict:
        """Handle for one producer process; it maps this ring's memory when turned into a ``RemoteRing``."""
        return {"memory": self._symm.export(), "layout": self.layout.to_dict(), "slots": self.slots,
                "run_id": self.run_id, "attempt_id": self.attempt_id, "consumer": self.consumer}

    def read(self, key: str, device_flags: bool = False, wait_limit_ms: float = 2000.0) -> Dict[str, torch.Tensor]:
        """Zero-copy views of a published sample.  Rejects descriptors of another run / attempt / consumer."""
        d = FeatureDescriptor.from_key(key)
        if d.run_id != self.run_id or d.attempt_id != self.attempt_id:
            raise RuntimeError(f"stale feature descriptor: run {d.run_id}/{d.attempt_id}, ring {self.run_id}/{self.attempt_id}")
        if d.consumer != self.consumer:
            raise RuntimeError(f"descriptor is addressed to consumer {d.consumer}, this ring is {self.consumer}")
        if device_flags and self.buffer.is_cuda:
            from aspec_b200 import _native
            rc = _native.kernels().ab_flag_wait(C.c_void_p(self.flags[d.slot:].data_ptr()), C.c_longlong(d.generation),
                                                C.c_double(wait_limit_ms), C.c_void_p(self.status.data_ptr()),
                                                C.c_void_p(torch.cuda.current_stream(self.buffer.device).cuda_stream))
            if rc != 0:
                raise RuntimeError(f"ab_flag_wait refused the launch ({rc})")
        elif device_flags and int(self.flags[d.slot]) < d.generation:
            raise TimeoutError("feature slot was not published")
        views = self.views(d.slot, d.n_tokens)
        if d.view_end is not None or d.view_start:
            end = d.n_tokens if d.view_end is None else d.view_end
            views = {k: v[d.view_start:end] for k, v in views.items()}
        return views

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise TimeoutError(f"waiting for a feature slot ran out of time (status {code})")


class RemoteRing(_SlotViews):
    """Producer side: the consumer's ring mapped into this process."""

    def __init__(self, handle: dict):
        from aspec_b200.parallel.symmetric_memory import SymmetricBuffer
        layout = SlotLayout(**handle["layout"])
        slots = handle["slots"]
        # mapped with this process's GPU current: the ring then looks like local memory to torch and to
        # the kernels, and every access crosses NVLink
        self._symm = SymmetricBuffer.open(handle["memory"])
        raw = self._symm.tensor
        payload = slots * layout.slot_bytes
        super().__init__(raw[:payload], raw[payload:payload + slots * 8].view(torch.int64), layout, slots)
        self.run_id, self.attempt_id, self.consumer = handle["run_id"], handle["attempt_id"], handle["consumer"]

    def descriptor(self, slot: int, generation: int, n_tokens: int, layer_ids) -> FeatureDescriptor:
        return FeatureDescriptor(self.run_id, self.attempt_id, self.consumer, slot, generation, n_tokens,
                                 tuple(layer_ids), self.layout.hidden, self.layout.dtype)

    def publish(self, slot: int, generation: int) -> None:
        """Make the slot's generation visible to the consumer (device-ordered on CUDA)."""
        if self.flags.is_cuda:
            from aspec_b200 import _native
            dev = torch.cuda.current_device()
            rc = _native.kernels().ab_flag_publish(C.c_void_p(self.flags[slot:].data_ptr()), C.c_longlong(generation),
                                                   C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
            if rc != 0:
                raise RuntimeError(f"ab_flag_publish refused the launch ({rc})")
        else:
            self.flags[slot] = generation


class RingFeatureSink:
    """``models.target.dense.FeatureSink`` protocol over one or several remote slots (multi-reader fan-out)."""

    def __init__(self, slot_views, layer_ids, hidden: int, reader_layer_ids=None):
        self.slot_views = list(slot_views)       # one dict of views per reader
        self.layer_ids = list(layer_ids)         # every layer the Target captures (union over readers)
        # readers of a shared Target may each want a subset of the captured layers, in their own column order
        self.reader_layer_ids = [list(r) for r in reader_layer_ids] if reader_layer_ids else [self.layer_ids] * len(self.slot_views)
        self.hidden = hidden
        self.hidden_states = self.slot_views[0]["hidden_states"]
        self.last_hidden_states = self.slot_views[0].get("last_hidden_states")

    def layer_views(self, layer_id: int):
        out = []
        for v, layers in zip(self.slot_views, self.reader_layer_ids):
            if layer_id in layers:
                col = layers.index(layer_id)
                out.append(v["hidden_states"][:, col * self.hidden:(col + 1) * self.hidden])
        return out

    def final_views(self):
        return [v["last_hidden_states"] for v in self.slot_views if "last_hidden_states" in v]
