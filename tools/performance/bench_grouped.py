"""``python -m tools.performance.bench_grouped``: SwiGLU expert bank forward + backward, grouped launches against the
per-expert loop of dense GEMMs (both on the tcgen05 kernels of this package).  CUDA events, L2 flushed between
iterations; prints one JSON line with times and the fraction of the measured GEMM peak."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--tokens", type=int, default=32768, help="routed rows (tokens x top-k)")
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--intermediate", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=8)
    args = ap.parse_args()
    from aspec_b200.ops.activation import swiglu
    from aspec_b200.ops.gemm import check_status
    from aspec_b200.ops.grouped_gemm import grouped_experts
    from aspec_b200.ops.linear import linear
    dev = torch.device("cuda")
    E, D, I, N = args.experts, args.hidden, args.intermediate, args.tokens
    g = torch.Generator().manual_seed(0)
    counts = torch.bincount(torch.randint(0, E, (N,), generator=g), minlength=E).tolist()
    bf = torch.bfloat16
    x = torch.randn(N, D, device=dev).to(bf).requires_grad_(True)
    gu = (torch.randn(E, 2 * I, D, device=dev) * 0.02).to(bf).requires_grad_(True)
    dn = (torch.randn(E, D, I, device=dev) * 0.02).to(bf).requires_grad_(True)
    dy = torch.randn(N, D, device=dev).to(bf)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def loop():
        outs, off = [], 0
        for e, n in enumerate(counts):
            if n:
                outs.append(linear(swiglu(linear(x[off:off + n], gu[e]), 0.0), dn[e]))
            off += n
        torch.cat(outs).backward(dy)

    def grouped():
        grouped_experts(x, gu, dn, counts).backward(dy)

    def timed(fn):
        best = float("inf")
        for it in range(args.iters + 3):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if it >= 3:
                best = min(best, a.elapsed_time(b))
            x.grad = gu.grad = dn.grad = None
        return best

    t_group, t_loop = timed(grouped), timed(loop)
    check_status(dev)
    flops = 3 * 2 * N * D * 3 * I                     # forward + two backward products of both projections
    peaks = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak = json.loads(peaks.read_text()).get("bf16_tflops", 1590.0) if peaks.exists() else 1590.0
    print(json.dumps({"case": "swiglu expert bank fwd+bwd", "rows": N, "experts": E, "hidden": D, "intermediate": I,
                      "grouped_ms": t_group, "loop_ms": t_loop, "grouped_tflops": flops / t_group / 1e9,
                      "frac_of_measured_gemm_peak": flops / t_group / 1e9 / peak}))


if __name__ == "__main__":
    main()
