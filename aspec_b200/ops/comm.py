"""Python face of the peer-memory communication kernels (``csrc/comm_sm100.cu``).

All functions take *lists of tensors that live on (or are mapped into) the launching GPU's address space*: a
tensor opened through ``parallel.symmetric_memory.SymmetricBuffer.open`` is peer HBM that looks local, so the same
call works for one process emulating several ranks on one GPU (tests) and for real multi-GPU peers.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from aspec_b200 import _native


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptrs(tensors: Sequence[torch.Tensor]):
    arr = (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} refused the launch (code {rc})")


def peer_reduce(peers: Sequence[torch.Tensor], out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``out = scale * sum(peers)`` (bf16 or fp32; element count a multiple of 8 / 4)."""
    _check(_native.kernels().ab_peer_reduce(_ptrs(peers), len(peers), C.c_void_p(out.data_ptr()), C.c_longlong(out.numel()),
                                            C.c_float(scale), int(out.dtype == torch.float32), _stream(out)), "ab_peer_reduce")
    return out


def shard_reduce_sumsq(peer_grads: Sequence[torch.Tensor], lo: int, shard: torch.Tensor, ctrl: torch.Tensor) -> None:
    """``shard = sum_r peer_grads[r][lo : lo + len(shard)]``; ``ctrl[0] += sum(shard^2)``, ``ctrl[1] += non-finite``."""
    _check(_native.kernels().ab_shard_reduce_sumsq(_ptrs(peer_grads), len(peer_grads), C.c_longlong(lo),
                                                   C.c_void_p(shard.data_ptr()), C.c_longlong(shard.numel()),
                                                   C.c_void_p(ctrl.data_ptr()), _stream(shard)), "ab_shard_reduce_sumsq")


def shard_adamw_scatter(master, grad, m, v, peer_params: Sequence[torch.Tensor], lo: int, ctrl, *, lr, beta1, beta2, eps,
                        wd, step, max_norm) -> None:
    """AdamW on the owned shard; the new bf16 weights are stored into every replica ``peer_params[r][lo : lo + n]``.
    ``step=None`` takes the bias-correction step from ``ctrl[4]`` (applied updates, counted on the device)."""
    f = C.c_float
    _check(_native.kernels().ab_shard_adamw_scatter(
        C.c_void_p(master.data_ptr()), C.c_void_p(grad.data_ptr()), C.c_void_p(m.data_ptr()), C.c_void_p(v.data_ptr()),
        _ptrs(peer_params), len(peer_params), C.c_longlong(lo), C.c_longlong(master.numel()), C.c_void_p(ctrl.data_ptr()),
        f(lr), f(beta1), f(beta2), f(eps), f(wd), f(0.0 if step is None else 1.0 - beta1 ** step),
        f(0.0 if step is None else 1.0 - beta2 ** step), f(max_norm),
        _stream(master)), "ab_shard_adamw_scatter")


def flags_signal(peer_flags: Sequence[torch.Tensor], index: int, value: int, stream=None) -> None:
    """Store ``value`` (release, system scope) into element ``index`` of every rank's int64 flag array."""
    st = C.c_void_p(stream.cuda_stream) if stream is not None else _stream(peer_flags[0])
    _check(_native.kernels().ab_flags_signal(_ptrs(peer_flags), len(peer_flags), C.c_longlong(index), C.c_longlong(value), st),
           "ab_flags_signal")


def flags_wait_all(flags: torch.Tensor, first: int, count: int, value: int, status: torch.Tensor, limit_ms: float = 5000.0,
                   stream=None) -> None:
    """Stream-ordered bounded wait until ``flags[first : first + count] >= value``; on expiry ``status`` holds the
    peer-timeout code and the stream continues (the host reads ``status`` at the end of the update)."""
    st = C.c_void_p(stream.cuda_stream) if stream is not None else _stream(flags)
    _check(_native.kernels().ab_flags_wait_all(C.c_void_p(flags.data_ptr() + 8 * first), count, C.c_longlong(value),
                                               C.c_double(limit_ms), C.c_void_p(status.data_ptr()), st), "ab_flags_wait_all")


def peer_gather(peer_shards: Sequence[torch.Tensor], dst: torch.Tensor, stream=None) -> None:
    """``dst = cat(peer_shards)`` by peer loads (every shard the same byte size, a multiple of 16)."""
    nbytes = peer_shards[0].numel() * peer_shards[0].element_size()
    st = C.c_void_p(stream.cuda_stream) if stream is not None else _stream(dst)
    _check(_native.kernels().ab_peer_gather(_ptrs(peer_shards), len(peer_shards), C.c_longlong(nbytes),
                                            C.c_void_p(dst.data_ptr()), st), "ab_peer_gather")


def shard_reduce_accum(peer_grads: Sequence[torch.Tensor], lo: int, shard: torch.Tensor, stream=None) -> None:
    """``shard += sum_r peer_grads[r][lo : lo + len(shard)]`` (fp32)."""
    st = C.c_void_p(stream.cuda_stream) if stream is not None else _stream(shard)
    _check(_native.kernels().ab_shard_reduce_accum(_ptrs(peer_grads), len(peer_grads), C.c_longlong(lo),
                                                   C.c_void_p(shard.data_ptr()), C.c_longlong(shard.numel()), st),
           "ab_shard_reduce_accum")


def peer_lse_merge(peer_lse: Sequence[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """``out[i] = logsumexp_r peer_lse[r][i]`` (fp32)."""
    _check(_native.kernels().ab_peer_lse_merge(_ptrs(peer_lse), len(peer_lse), C.c_void_p(out.data_ptr()),
                                               C.c_longlong(out.numel()), _stream(out)), "ab_peer_lse_merge")
    return out


def peer_argmax_merge(peer_vals: Sequence[torch.Tensor], peer_idxs: Sequence[torch.Tensor], labels: torch.Tensor,
                      correct: torch.Tensor) -> torch.Tensor:
    """``correct[i] = (argmax over all shards == labels[i])``; ``peer_idxs`` hold global column indices (int32)."""
    _check(_native.kernels().ab_peer_argmax_merge(_ptrs(peer_vals), _ptrs(peer_idxs), len(peer_vals),
                                                  C.c_void_p(labels.data_ptr()), C.c_void_p(correct.data_ptr()),
                                                  C.c_longlong(correct.numel()), _stream(correct)), "ab_peer_argmax_merge")
    return correct


def attn_merge_partials(part_o: torch.Tensor, part_lse: torch.Tensor, n_rows: int, out: torch.Tensor, lse_out: torch.Tensor) -> None:
    """``part_o [P, R_max, H, d]`` (bf16) and ``part_lse [P, H * R_max]`` (fp32, each part holding ``[H, n_rows]`` in its
    first ``H * n_rows`` entries) -> ``out [n_rows, H, d]``, ``lse_out [H, n_rows]``: the exact merge of attention
    partials over disjoint key sets in one kernel (``ops.attention.merge_partials`` is the fp32 statement)."""
    P, _, H, d = part_o.shape
    rc = _native.kernels().ab_attn_merge_partials(
        C.c_void_p(part_o.data_ptr()), C.c_longlong(part_o.stride(0)), C.c_void_p(part_lse.data_ptr()),
        C.c_longlong(part_lse.stride(0)), C.c_int(P), C.c_int(n_rows), C.c_int(H), C.c_int(d),
        C.c_void_p(out.data_ptr()), C.c_void_p(lse_out.data_ptr()), C.c_float(float("-inf")), _stream(part_o))
    _check(rc, "ab_attn_merge_partials")
