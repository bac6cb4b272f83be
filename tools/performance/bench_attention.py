"""Attention micro-benchmark on the reference's published SM100 workload (docs/dspark_attn_kernel_optimization.md:55-63,
tools/performance/benchmark_cudnn_gqa.py:19-85): 12 packed documents ``[4096] * 10 + [40960, 49152]``, 512 random
anchors per document, block 7 -> Q ``[43008, 32, 128]``, K/V ``[174080, 8, 128]`` bf16.  Published on an SM100 GPU:
18.12 ms forward + backward (4.47 + 12.93) for cuDNN forward + the joint-GQA CuTe-DSL backward.

``python -m tools.performance.bench_attention [--iters N] [--small]`` prints one JSON line: forward / backward ms
(CUDA events, L2 flushed between iterations) and the algorithmic FLOP rate.
"""
from __future__ import annotations

import argparse
import json

import torch


def workload(small: bool = False, seed: int = 1019):
    from aspec_b200.ops.attention import build_block_intervals
    docs = [512] * 3 + [2048] if small else [4096] * 10 + [40960, 49152]
    n_anchor, bs, hq, hkv, d = (64 if small else 512), 7, 32, 8, 128
    g = torch.Generator().manual_seed(seed)
    anchors, starts, off = [], [], 0
    for i, n in enumerate(docs):
        a = torch.sort(torch.randint(1, n - bs, (n_anchor,), generator=torch.Generator().manual_seed(20261031 + i))).values
        anchors.append(a + off)
        starts.append(torch.full((n_anchor,), off))
        off += n
    anchors, starts = torch.cat(anchors), torch.cat(starts)
    T = off
    iv = build_block_intervals(anchors, torch.ones_like(anchors, dtype=torch.bool), ctx_len=T, block_size=bs, doc_start=starts).cuda()
    Q = anchors.numel() * bs
    mk = lambda *s: (torch.randn(*s, generator=g) * 1.0).to(torch.bfloat16).cuda()
    q, k, v, do = mk(Q, hq, d), mk(T + Q, hkv, d), mk(T + Q, hkv, d), mk(Q, hq, d)
    visible = ((iv[:, 1] - iv[:, 0]) + (iv[:, 3] - iv[:, 2])).sum().item()
    return q, k, v, do, iv, visible


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args()
    from aspec_b200.ops import attention_sm100 as A
    from aspec_b200.ops.gemm import check_status
    q, k, v, do, iv, visible = workload(a.small)
    scale = 128 ** -0.5
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
    out, lse = A.forward(q, k, v, iv, scale)
    for _ in range(3):
        A.forward(q, k, v, iv, scale)
        A.backward(q, k, v, iv, out, lse, do, scale)
    tf = tb = 0.0
    for _ in range(a.iters):
        flush.add_(1)
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        out, lse = A.forward(q, k, v, iv, scale)
        e[1].record()
        A.backward(q, k, v, iv, out, lse, do, scale)
        e[2].record()
        torch.cuda.synchronize()
        tf += e[0].elapsed_time(e[1])
        tb += e[1].elapsed_time(e[2])
    check_status("cuda")
    tf, tb = tf / a.iters, tb / a.iters
    hq, d = q.shape[1], q.shape[2]
    fwd_flops = 4.0 * visible * hq * d
    print(json.dumps({"workload": "reference SM100 attention micro-benchmark" + (" (small)" if a.small else ""),
                      "q_rows": q.shape[0], "kv_rows": k.shape[0], "visible_pairs": visible, "fwd_ms": tf, "bwd_ms": tb,
                      "total_ms": tf + tb, "published_total_ms": 18.12, "published_fwd_ms": 4.47, "published_bwd_ms": 12.93,
                      "fwd_tflops": fwd_flops / tf / 1e9, "bwd_tflops": 2.5 * fwd_flops / tb / 1e9}))


if __name__ == "__main__":
    main()
