"""Peer-memory primitives on one GPU: device flags with bounded waits (a wait on a flag that nothing sets runs out
and reports a status; the context stays usable), byte copies and peer reductions."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def test_flag_wait_times_out_with_a_status_and_the_context_survives():
    from aspec_b200 import _native
    lib = _native.kernels()
    dev = torch.device("cuda:0")
    flag = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # nothing ever publishes generation 5: the wait must give up after ~50 ms and record "peer timeout"
    rc = lib.ab_flag_wait(C.c_void_p(flag.data_ptr()), C.c_longlong(5), C.c_double(50.0), C.c_void_p(status.data_ptr()), _stream(dev))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 3
    # waits longer than the library's cap are refused on the host
    assert lib.ab_flag_wait(C.c_void_p(flag.data_ptr()), C.c_longlong(5), C.c_double(60000.0), C.c_void_p(status.data_ptr()), _stream(dev)) == -10
    # a published flag satisfies the wait immediately and the device still works
    status.zero_()
    assert lib.ab_flag_publish(C.c_void_p(flag.data_ptr()), C.c_longlong(7), _stream(dev)) == 0
    assert lib.ab_flag_wait(C.c_void_p(flag.data_ptr()), C.c_longlong(7), C.c_double(50.0), C.c_void_p(status.data_ptr()), _stream(dev)) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(flag.item()) == 7
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0


def test_peer_reduce_and_lse_merge():
    from aspec_b200.ops import comm
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    parts = [torch.randn(4096, device=dev) for _ in range(3)]
    out = comm.peer_reduce(parts, torch.empty(4096, device=dev), scale=0.5)
    assert torch.allclose(out, 0.5 * sum(parts), atol=1e-6)
    bparts = [torch.randn(4096, device=dev).bfloat16() for _ in range(4)]
    bout = comm.peer_reduce(bparts, torch.empty(4096, device=dev, dtype=torch.bfloat16))
    assert torch.allclose(bout.float(), sum(p.float() for p in bparts), atol=3e-2)
    lses = [torch.randn(1000, device=dev) * 3 for _ in range(3)]
    lses[1][::7] = float("-inf")
    merged = comm.peer_lse_merge(lses, torch.empty(1000, device=dev))
    assert torch.allclose(merged, torch.logsumexp(torch.stack(lses), 0), atol=1e-5)
    vals = [torch.randn(500, device=dev) for _ in range(2)]
    idxs = [torch.randint(0, 100, (500,), device=dev, dtype=torch.int32), torch.randint(100, 200, (500,), device=dev, dtype=torch.int32)]
    want = torch.where(vals[0] >= vals[1], idxs[0], idxs[1]).long()
    correct = comm.peer_argmax_merge(vals, idxs, want, torch.empty(500, device=dev))
    assert bool((correct == 1).all())
