"""Sparse-attention micro-benchmark at the long-context DSA shape: one 64 K-token document, 512 anchors x block 7 =
3584 draft queries, 32 / 8 heads of 128, a lightning indexer with 64 heads of 128, top-k 2048.

``python -m tools.performance.bench_sparse [--context 65536] [--topk 2048] [--iters 5] [--small]`` prints one JSON line
with CUDA-event times (L2 flushed between iterations) and each kernel's fraction of its roofline, against the pool's
measured peaks (``MEASURED_PEAKS.json`` at the repository root when present; else 6.65 TB/s and 1.59 PFLOP/s):

* indexer scores - a GEMM: ``2 * H * d`` FLOPs per eligible (query, key) pair against the measured cuBLAS bf16 rate;
* top-k - five passes over the eligible scores (four radix passes + the ordered output pass) against copy bandwidth;
* selected-key attention forward / backward - gathers ``2 x 256`` bytes per (query, key/value head, selected key);
  the denominator is copy bandwidth (most gathers hit L2, so a fraction above 1 is possible).
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return m["hbm_gbs"], m["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=65536)
    ap.add_argument("--anchors", type=int, default=512)
    ap.add_argument("--topk", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args()
    if a.small:
        a.context, a.anchors, a.topk = 4096, 64, 256
    from aspec_b200.ops import sparse_attention as SA
    from aspec_b200.ops.gemm import check_status
    T, bs, hq, hkv, d, H = a.context, 7, 32, 8, 128, 64
    g = torch.Generator().manual_seed(0)
    anchors = torch.sort(torch.randint(T // 4, T - bs, (a.anchors,), generator=g)).values
    n = a.anchors * bs
    lo = torch.zeros(n, dtype=torch.int32, device="cuda")
    hi = anchors.repeat_interleave(bs).to(torch.int32).cuda()
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    q, k, v, do = mk(n, hq, d), mk(T + n, hkv, d), mk(T + n, hkv, d), mk(n, hq, d)
    qi, ki = mk(n, H, d), mk(T, d)
    w = (torch.rand(n, H, generator=g) * 0.1).cuda()
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
    own = (T + torch.arange(n, device="cuda").view(-1, bs)[:, :1] + torch.arange(bs, device="cuda")[None]).repeat_interleave(bs, 0)

    def timed(fn):
        fn()
        total = 0.0
        for _ in range(a.iters):
            flush.add_(1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / a.iters, out

    t_scores_one, _ = timed(lambda: SA.indexer_scores(qi, ki, w, lo, hi, epilogue_groups=1))
    t_scores, scores = timed(lambda: SA.indexer_scores(qi, ki, w, lo, hi))
    t_topk, sel = timed(lambda: SA.topk_select(scores, lo, hi, a.topk))
    sel_full = torch.cat([sel, own.to(torch.int32)], 1).contiguous()
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    t_fwd, (out, lse) = timed(lambda: SA.selected_attention(q, k, v, sel_full, d ** -0.5))

    def bwd():
        q.grad = k.grad = v.grad = None
        out.backward(do, retain_graph=True)
    t_bwd, _ = timed(bwd)
    check_status("cuda")
    hbm, tflops, kind = _peaks()
    pairs = float((hi - lo).clamp(min=0).sum())
    L = sel_full.shape[1]
    sel_n = float((sel_full >= 0).sum())
    res = {
        "workload": f"DSA sparse stage, context {T}, {n} queries, top-k {a.topk} + {bs} own-block keys, {hq}/{hkv} heads",
        "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "kind": kind},
        "indexer_scores_ms_one_epilogue_warpgroup": t_scores_one, "indexer_scores_ms": t_scores, "indexer_tflops": 2.0 * H * d * pairs / t_scores / 1e9,
        "topk_ms": t_topk, "topk_gbs": 5 * 4 * pairs / t_topk / 1e6,
        "selected_attention_fwd_ms": t_fwd, "fwd_gather_gbs": sel_n * hkv * 2 * 256 / t_fwd / 1e6,
        "selected_attention_bwd_ms": t_bwd, "bwd_gather_plus_reduce_gbs": sel_n * hkv * (2 * 256 + 2 * 512) / t_bwd / 1e6,
        "list_length": L,
    }
    res["indexer_fraction_of_" + kind] = res["indexer_tflops"] / tflops
    res["topk_fraction_of_" + kind] = res["topk_gbs"] / hbm
    res["fwd_fraction_of_" + kind] = res["fwd_gather_gbs"] / hbm
    res["bwd_fraction_of_" + kind] = res["bwd_gather_plus_reduce_gbs"] / hbm
    print(json.dumps(res))


if __name__ == "__main__":
    main()
