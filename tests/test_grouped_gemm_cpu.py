"""Tile / segment tables of the grouped GEMM, executed by a CPU interpreter of the kernel's contract.

The tables are what the kernel consumes; interpreting them with plain tensor arithmetic checks the planning code (row
offsets, padded layouts, multi-source reductions, masked edges) without a GPU."""
import numpy as np
import torch

from aspec_b200.ops import grouped_gemm as G


def _interpret(operands, tiles, segs, a_mn, b_mn, fp32, alpha, outputs):
    """Apply the kernel's semantics: D_t[:rows, :cols] = alpha * sum_seg A_seg[128, 64 k] @ B_seg[256, 64 k]^T with rows
    past a tensor's end reading as zero (the TMA fill)."""
    def block(t, r0, nr, c0, nc):
        out = torch.zeros(nr, nc)
        r1, c1 = min(r0 + nr, t.shape[0]), min(c0 + nc, t.shape[1])
        if r1 > r0 and c1 > c0:
            out[: r1 - r0, : c1 - c0] = t[r0:r1, c0:c1].float()
        return out

    for tile in tiles:
        acc = torch.zeros(G.BM, G.BN)
        for sg in segs[tile["seg0"]: tile["seg0"] + tile["nseg"]]:
            k = int(sg["k_blocks"]) * G.BK
            a_t, b_t = operands[sg["a_map"]][0], operands[sg["b_map"]][0]
            a = block(a_t, sg["a_k"], k, sg["a_mn"], G.BM).t() if a_mn else block(a_t, sg["a_mn"], G.BM, sg["a_k"], k)
            b = block(b_t, sg["b_k"], k, sg["b_mn"], G.BN).t() if b_mn else block(b_t, sg["b_mn"], G.BN, sg["b_k"], k)
            acc += a @ b.t()
        ptr = int(tile["d"])
        for o in outputs:                                   # locate the destination tensor of this tile
            base, size = o.data_ptr(), o.numel() * o.element_size()
            if base <= ptr < base + size:
                flat = o.view(-1)
                start = (ptr - base) // o.element_size()
                for r in range(int(tile["rows"])):
                    row = start + r * int(tile["ldd"])
                    flat[row: row + int(tile["cols"])] = (alpha * acc[r, : int(tile["cols"])]).to(o.dtype)
                break
        else:
            raise AssertionError("tile points outside every output buffer")


def _patched(monkeypatch, outputs):
    def fake(operands, tiles, segs, a_mn, b_mn, fp32, alpha, device, max_ctas=0):
        _interpret(operands, tiles, segs, a_mn, b_mn, fp32, alpha, outputs)
    monkeypatch.setattr(G, "_launch", fake)


def test_rows_plan_matches_per_problem_products(monkeypatch):
    torch.manual_seed(0)
    E, N, K = 3, 320, 192
    a0, a1 = torch.randn(300, K).bfloat16(), torch.randn(200, K).bfloat16()
    for b_t in (False, True):
        w = (torch.randn(E, K, N) if b_t else torch.randn(E, N, K)).bfloat16()
        o0, o1 = torch.full((400, N), 7.0).bfloat16(), torch.full((300, N + 8), 7.0).bfloat16()
        _patched(monkeypatch, [o0, o1])
        src, a_row, rows, expert, dst, out_row = [0, 1, 0, 1], [3, 0, 200, 150], [150, 129, 0, 50], [0, 1, 2, 2], [0, 0, 1, 1], [0, 150, 0, 17]
        G.rows_gemm([a0, a1], w, [o0, o1], src=src, a_row=a_row, rows=rows, expert=expert, dst=dst, out_row=out_row, b_t=b_t)
        e0, e1 = torch.full((400, N), 7.0), torch.full((300, N + 8), 7.0)
        for s, ar, n, e, d, orow in zip(src, a_row, rows, expert, dst, out_row):
            wm = w[e].float() if b_t else w[e].float().t()
            (e0, e1)[d][orow:orow + n, :N] = (a0, a1)[s][ar:ar + n].float() @ wm
        assert torch.allclose(o0.float(), e0, atol=0.3, rtol=0.02) and torch.allclose(o1.float(), e1, atol=0.3, rtol=0.02)


def test_wgrad_plan_reduces_over_sources_with_a_padded_operand(monkeypatch):
    torch.manual_seed(1)
    E, Ma, Nb = 3, 192, 320
    counts = [[70, 0, 130], [1, 0, 64]]
    a_bufs = [torch.randn(sum(c), Ma).bfloat16() for c in counts]
    runs = [(s, e, counts[s][e]) for s in range(2) for e in range(E)]
    pstart, ptotal = G.padded_offsets([n for _, _, n in runs])
    assert all(p % 64 == 0 for p in pstart) and ptotal % 64 == 0
    b = torch.zeros(ptotal, Nb).bfloat16()
    ref = torch.zeros(E, Ma, Nb)
    a_row = []
    for (s, e, n), p0 in zip(runs, pstart):
        o = sum(counts[s][:e])
        a_row.append(o)
        blk = torch.randn(n, Nb).bfloat16()
        b[p0:p0 + n] = blk
        ref[e] += a_bufs[s][o:o + n].float().t() @ blk.float()
    out = torch.full((E, Ma, Nb), 3.0)
    _patched(monkeypatch, [out])
    G.wgrad_gemm(a_bufs, [b], out, expert=[e for _, e, _ in runs], a_src=[s for s, _, _ in runs], a_row=a_row,
                 b_src=[0] * len(runs), b_row=pstart, rows=[n for _, _, n in runs])
    assert torch.equal(out[1], torch.zeros(Ma, Nb))             # an expert without rows is zero-filled, not skipped
    assert torch.allclose(out, ref, atol=1e-2, rtol=1e-3)


def test_native_planner_writes_the_same_tables_as_the_array_statement(monkeypatch):
    """The C++ planner (runtime library) against the numpy planner, table for table."""
    rng = np.random.default_rng(0)
    captured = {}

    def capture(key):
        def fake(operands, tiles, segs, *rest, **kw):
            captured[key] = (tiles.copy(), segs.copy())
        return fake

    E, N, K = 7, 600, 200
    a_bufs = [torch.zeros(4000, K).bfloat16(), torch.zeros(3000, K).bfloat16()]
    outs = [torch.zeros(5000, N).bfloat16(), torch.zeros(5000, N + 8).bfloat16()]
    n = 40
    rows = rng.integers(0, 300, n)
    rows[::7] = 0
    args = dict(src=rng.integers(0, 2, n), a_row=rng.integers(0, 2000, n), rows=rows, expert=rng.integers(0, E, n),
                dst=rng.integers(0, 2, n), out_row=rng.integers(0, 3000, n))
    for b_t in (False, True):
        w = torch.zeros((E, K if b_t else N, N if b_t else K)).bfloat16() if not b_t else torch.zeros(E, 192, N).bfloat16()
        bufs = a_bufs if not b_t else [torch.zeros(4000, 192).bfloat16(), torch.zeros(3000, 192).bfloat16()]
        for native in (True, False):
            monkeypatch.setattr(G, "NATIVE_PLANNER", native)
            monkeypatch.setattr(G, "_launch", capture(native))
            G.rows_gemm(bufs, w, outs, b_t=b_t, **args)
        for a, b in zip(captured[True], captured[False]):
            assert a.dtype == b.dtype and a.tobytes() == b.tobytes()
    out = torch.zeros(E, 300, 520)
    runs = 25
    wargs = dict(expert=rng.integers(0, E, runs), a_src=rng.integers(0, 2, runs), a_row=rng.integers(0, 2000, runs),
                 b_src=np.zeros(runs, dtype=np.int64), b_row=rng.integers(0, 30, runs) * 64, rows=rng.integers(0, 200, runs))
    for native in (True, False):
        monkeypatch.setattr(G, "NATIVE_PLANNER", native)
        monkeypatch.setattr(G, "_launch", capture(native))
        G.wgrad_gemm([torch.zeros(4000, 300).bfloat16(), torch.zeros(3000, 300).bfloat16()], [torch.zeros(4000, 520).bfloat16()], out, **wargs)
    for a, b in zip(captured[True], captured[False]):
        assert a.tobytes() == b.tobytes()
