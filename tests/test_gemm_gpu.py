"""tcgen05 GEMM against a float32 PyTorch reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().t()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 300, 136), (1024, 1536, 4096)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_t, b_t):
    from aspec_b200.ops import gemm as G
    torch.manual_seed(0)
    # leading dimensions must be multiples of 8 elements: pad storage, slice the view
    def mk(r, c):
        cp = (c + 7) // 8 * 8
        return (torch.randn(r, cp, device="cuda") * 0.5).bfloat16()[:, :c]
    a = mk(M, K)
    b = mk(N, K)
    a_arg = a.t().contiguous() if a_t else a
    b_arg = b.t().contiguous() if b_t else b
    if a_t and M % 8:
        pytest.skip("MN-major operand needs MN extent multiple of 8")
    if b_t and N % 8:
        pytest.skip("MN-major operand needs MN extent multiple of 8")
    out = G.gemm(a_arg, b_arg, a_t=a_t, b_t=b_t)
    G.check_status("cuda")
    ref = _ref(a, b)
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * (K ** 0.5) * 0.25 + 1e-2
    assert err < tol, f"max err {err} (tol {tol})"


def test_gemm_fp32_out_addend_dual():
    from aspec_b200.ops import gemm as G
    torch.manual_seed(1)
    M, N, K, K2 = 384, 512, 512, 256
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    a2 = (torch.randn(M, K2, device="cuda") * 0.3).bfloat16()
    b2 = (torch.randn(N, K2, device="cuda") * 0.3).bfloat16()
    c = torch.randn(M, N, device="cuda")
    out = G.gemm(a, b, a2=a2, b2=b2, out_dtype=torch.float32, addend=c, alpha=0.5)
    G.check_status("cuda")
    ref = 0.5 * (_ref(a, b) + _ref(a2, b2)) + c
    assert (out - ref).abs().max().item() < 2e-2


def test_gemm_rowstats():
    from aspec_b200.ops import gemm as G
    torch.manual_seed(2)
    M, N, K = 300, 1000, 256
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    nt = (N + G.TILE_N - 1) // G.TILE_N
    stats = torch.zeros(nt, M, 2, device="cuda")
    logits = G.gemm(a, b, epilogue=G.EPI_ROWSTATS, stats=stats)
    G.check_status("cuda")
    ref = _ref(a, b)
    assert (logits.float() - ref).abs().max().item() < 5e-2
    lse = torch.logsumexp(stats[..., 0] + torch.log(stats[..., 1]), dim=0)
    ref_lse = torch.logsumexp(logits.float(), dim=1)
    assert (lse - ref_lse).abs().max().item() < 1e-3


def test_gemm_swiglu():
    from aspec_b200.ops import gemm as G
    torch.manual_seed(3)
    M, I, K = 256, 384, 256
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    wg = (torch.randn(I, K, device="cuda") * 0.1).bfloat16()
    wu = (torch.randn(I, K, device="cuda") * 0.1).bfloat16()
    # interleave in blocks of 128 rows: [gate block, up block] per 256-row tile
    w = torch.stack([wg.view(I // 128, 128, K), wu.view(I // 128, 128, K)], 1).reshape(2 * I, K).contiguous()
    out = G.gemm(x, w, epilogue=G.EPI_SWIGLU)
    G.check_status("cuda")
    g = _ref(x, wg)
    u = _ref(x, wu)
    ref = torch.nn.functional.silu(g) * u
    assert (out.float() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("M,N,K", [(384, 512, 2048), (3584, 4096, 1536), (200, 300, 1000)])
def test_gemm_stream_k(M, N, K):
    from aspec_b200.ops import gemm as G
    torch.manual_seed(5)
    Kp = (K + 7) // 8 * 8
    a = (torch.randn(M, Kp, device="cuda") * 0.2).bfloat16()[:, :K]
    b = (torch.randn(N, Kp, device="cuda") * 0.2).bfloat16()[:, :K]
    ref = _ref(a, b)
    out32 = G.gemm(a, b, out_dtype=torch.float32, stream_k=True)
    out16 = G.gemm(a, b, stream_k=True)
    acc = torch.ones(M, N, device="cuda")
    G.gemm(a, b, out=acc, addend=acc, out_dtype=torch.float32, stream_k=True)
    G.check_status("cuda")
    tol = 2e-2 * (K ** 0.5) * 0.1 + 1e-2
    assert (out32 - ref).abs().max().item() < tol
    assert (out16.float() - ref).abs().max().item() < tol + 0.05
    assert (acc - 1 - ref).abs().max().item() < tol


@pytest.mark.parametrize("M,N", [(300, 768), (257, 600)])
def test_gemm_mirrored_stores_match_the_primary_output(M, N):
    """Broadcast mirrors (with a residual addend): whole tiles take the shared-memory transposed store path, the
    ragged last column tile the per-thread path; rows past M are never written."""
    from aspec_b200.ops import gemm as G
    K = 192
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    mirrors = [torch.full((M + 5, N + 8), 9.0, device="cuda", dtype=torch.bfloat16)[:M, :N] for _ in range(3)]
    G.gemm(a, b, out=out, addend=res, mirrors=mirrors)
    G.check_status("cuda")
    ref = a.float() @ b.float().t() + res.float()
    assert torch.allclose(out.float(), ref, atol=0.15, rtol=0.02)
    for m in mirrors:
        assert torch.equal(m, out)
        base = m._base if m._base is not None else m
        assert torch.all(base[M:] == 9.0) and torch.all(base[:, N:] == 9.0)


def test_gemm_scatter_epilogue_splits_columns_over_destinations():
    from aspec_b200.ops import gemm as G
    M, K, per, n_dst = 200, 128, 256, 3
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(per * n_dst, K, device="cuda") * 0.5).bfloat16()
    dsts = [torch.full((M + 3, per), 5.0, device="cuda", dtype=torch.bfloat16) for _ in range(n_dst)]
    G.gemm(a, b, mirrors=[d[:M] for d in dsts], scatter_cols=per)
    G.check_status("cuda")
    ref = (a.float() @ b.float().t())
    for i, d in enumerate(dsts):
        assert torch.allclose(d[:M].float(), ref[:, i * per:(i + 1) * per], atol=0.1, rtol=0.02)
        assert torch.all(d[M:] == 5.0)


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True)])
def test_gemm_single_cta_and_cta_pair_kernels_agree(pair, a_t, b_t):
    """Both schedules of the kernel (one CTA per 128 x 256 tile; a cluster pair per 256 x 256 tile with
    ``cta_group::2`` MMAs) against the fp32 product, on a shape with ragged edges in M, N and K."""
    from aspec_b200.ops import gemm as G
    M, N, K = 392, 776, 328
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    out = G.gemm(a.t().contiguous() if a_t else a, b.t().contiguous() if b_t else b, a_t=a_t, b_t=b_t, cta_pair=pair)
    G.check_status("cuda")
    assert torch.allclose(out.float(), _ref(a, b), atol=0.2, rtol=0.02)
