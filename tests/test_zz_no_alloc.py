"""The allocation-free attention backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory themselves (a host program or serving
plug-in whose GPU memory is planned by another component).  For them ``ab_attn_bwd_static_scratch``
keeps its scratch in a fixed block inside the library.  This test loads the shared object with plain
``ctypes``, calls that symbol twice in a row on different inputs, and checks dQ / dK / dV against the
regular entry point (which takes caller-provided scratch), with the tolerance the other attention
tests use.  It also checks that an oversized problem is refused with the documented code.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, n_ctx, n_blocks, bs, hq, hkv):
    from aspec_b200.ops import attention_sm100 as K
    from aspec_b200.ops.attention import build_block_intervals
    g = torch.Generator().manual_seed(seed)
    anchors = torch.sort(torch.randint(1, n_ctx - bs, (n_blocks,), generator=g)).values
    keep = torch.rand(n_blocks, generator=g) > 0.1
    iv = build_block_intervals(anchors, keep, ctx_len=n_ctx, block_size=bs).cuda()
    Q = n_blocks * bs
    q = torch.randn(Q, hq, 128, generator=g).cuda().bfloat16()
    k = torch.randn(n_ctx + Q, hkv, 128, generator=g).cuda().bfloat16()
    v = torch.randn(n_ctx + Q, hkv, 128, generator=g).cuda().bfloat16()
    do = torch.randn(Q, hq, 128, generator=g).cuda().bfloat16()
    scale = 128 ** -0.5
    out, lse = K.forward(q, k, v, iv, scale)
    return q, k, v, iv, out, lse, do, scale


def _call_static(lib, q, k, v, iv, out, lse, do, scale):
    Q, hq, d = q.shape
    tk, hkv = k.shape[0], k.shape[1]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    rc = lib.ab_attn_bwd_static_scratch(
        p(q), p(k), p(v), p(iv), p(out), p(lse), p(do), p(dq), p(dk), p(dv), Q, tk, hq, hkv, d,
        C.c_longlong(k.stride(0)), C.c_longlong(v.stride(0)), C.c_float(scale), p(status),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, dq, dk, dv, int(status.item())


def test_static_scratch_backward_matches_regular_entry_point():
    from aspec_b200 import _native
    from aspec_b200.ops import attention_sm100 as K
    lib = C.CDLL(str(_native._KERNEL_LIB))
    lib.ab_attn_bwd_static_scratch.restype = C.c_int
    for seed, shape in ((11, (600, 40, 7, 8, 2)), (12, (333, 25, 4, 4, 1))):
        q, k, v, iv, out, lse, do, scale = _inputs(seed, *shape)
        rc, dq, dk, dv, status = _call_static(lib, q, k, v, iv, out, lse, do, scale)
        assert rc == 0 and status == 0
        rq, rk, rv = K.backward(q, k, v, iv, out, lse, do, scale)
        torch.cuda.synchronize()
        for name, a, b in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
            err = (a.float() - b.float()).abs().max().item()
            assert err < 6e-2 * max(1.0, b.float().abs().max().item()), f"{name} differs by {err}"


def test_static_scratch_refuses_sizes_beyond_its_block():
    from aspec_b200 import _native
    lib = C.CDLL(str(_native._KERNEL_LIB))
    lib.ab_attn_bwd_static_scratch.restype = C.c_int
    z = C.c_void_p(0)
    # hq * q_total = 32 * 100000 floats exceeds the 2 Mi-float block: refused before any launch
    rc = lib.ab_attn_bwd_static_scratch(z, z, z, z, z, z, z, z, z, z, 100000, 1000, 32, 8, 128,
                                        C.c_longlong(1024), C.c_longlong(1024), C.c_float(0.1), z, z)
    assert rc == -20
