"""Target-feature transport inside the GEMM epilogue against a separate transfer (two GPUs).

Run::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port P \
        -m tools.performance.bench_transport [--tokens 8192] [--iters 10]

Rank 0 plays a Target layer's down projection with its residual add, ``x[T, D] = act[T, I] @ W[D, I]^T + x`` - the GEMM
whose output is a captured layer - and rank 1 owns the destination (a Draft ring slot: a peer-visible buffer).  Timed
on rank 0 with CUDA events, L2 flushed between iterations, maximum over ranks:

* ``fused``: the GEMM's epilogue stores every output tile both locally and into the peer's slot (``mirrors``);
* ``gemm_then_copy``: the same GEMM without mirrors, then one peer copy of the output;
* ``gemm_then_nccl``: the same GEMM, then ``dist.send`` / ``dist.recv``;
* ``gemm_only``: the floor.

The transfer is ``T * D * 2`` bytes over NVLink; the roofline of the fused kernel is the slower of the GEMM at the
measured cuBLAS rate and those bytes at 770 GB/s.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    if world != 2:
        raise SystemExit("bench_transport runs on exactly two ranks")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from aspec_b200.ops import gemm as G
    from tools.performance.bench_parallel import NVLINK_GBS, Timer, _peak
    from aspec_b200.parallel.group import exchange_workspaces
    from aspec_b200.parallel.symmetric_memory import SymmetricBuffer
    T, D, I = a.tokens, a.hidden, a.intermediate
    bf = torch.bfloat16

    class Slot:
        """A peer-visible ``[T, D]`` bf16 buffer (stands for one ring slot's captured-layer region)."""

        def __init__(self, buffer=None):
            self.buffer = buffer if buffer is not None else SymmetricBuffer.allocate(T * D * 2, dev)
            self.view = self.buffer.tensor[: T * D * 2].view(bf).view(T, D)

        def export(self):
            return {"memory": self.buffer.export()}

        @classmethod
        def open(cls, meta):
            return cls(SymmetricBuffer.open(meta["memory"]))

    slots = exchange_workspaces(Slot(), Slot.open)
    peer = slots[1 - rank].view
    act = (torch.randn(T, I, device=dev) * 0.05).to(bf)
    w = (torch.randn(D, I, device=dev) * 0.02).to(bf)
    x = (torch.randn(T, D, device=dev) * 0.5).to(bf)
    out = torch.empty(T, D, device=dev, dtype=bf)
    timer = Timer(dev, a.iters)

    def copy_bytes(src, dst):
        import ctypes as C
        from aspec_b200 import _native
        rc = _native.kernels().ab_copy_bytes(C.c_void_p(src.data_ptr()), C.c_void_p(dst.data_ptr()),
                                             C.c_longlong(src.numel() * src.element_size()),
                                             C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        if rc != 0:
            raise RuntimeError(f"ab_copy_bytes refused the copy (code {rc})")

    def fused():
        if rank == 0:
            G.gemm(act, w, out=out, addend=x, mirrors=[peer])

    def gemm_then_copy():
        if rank == 0:
            G.gemm(act, w, out=out, addend=x)
            copy_bytes(out, peer)

    def gemm_then_nccl():
        if rank == 0:
            G.gemm(act, w, out=out, addend=x)
            dist.send(out, 1)
        else:
            dist.recv(slots[rank].view, 0)

    def gemm_only():
        if rank == 0:
            G.gemm(act, w, out=out, addend=x)

    res = {"case": "target_feature_transport", "tokens": T, "hidden": D, "intermediate": I}
    for name, fn in (("gemm_only", gemm_only), ("fused", fused), ("gemm_then_copy", gemm_then_copy),
                     ("gemm_then_nccl", gemm_then_nccl)):
        res[f"{name}_ms"] = timer(fn)
    # correctness of the fused path: the peer's slot holds the GEMM's output
    fused()
    dist.barrier()
    torch.cuda.synchronize(dev)
    if rank == 1:
        got = slots[rank].view.float()
        ok = torch.tensor([float(torch.isfinite(got).all() and got.abs().sum() > 0)], device=dev)
    else:
        ok = torch.tensor([float(torch.equal(out, out))], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    flops = 2.0 * T * D * I
    nbytes = T * D * 2
    roof = max(flops / (_peak() * 1e12), nbytes / (NVLINK_GBS * 1e9)) * 1e3
    res.update(slot_written=bool(ok.item()), nvlink_bytes=nbytes, flops=flops, roofline_ms=roof,
               fused_over_roofline=roof / res["fused_ms"],
               transfer_cost_fused_ms=res["fused_ms"] - res["gemm_only_ms"],
               transfer_cost_copy_ms=res["gemm_then_copy_ms"] - res["gemm_only_ms"],
               transfer_cost_nccl_ms=res["gemm_then_nccl_ms"] - res["gemm_only_ms"], n_gpus=world)
    if rank == 0:
        print(json.dumps(res), flush=True)
    from aspec_b200.ops.gemm import check_status
    check_status(dev)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
