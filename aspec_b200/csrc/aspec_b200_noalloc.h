// Entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference framework; it exists only in this library.
//
// Who needs it: programs that link the kernel library directly (a C or C++ host, a plug-in inside a
// serving process) and whose device memory is planned up front by someone else.  Such a caller
// typically may not call cudaMalloc at all: the owner of the memory pool has already reserved the
// device, an allocation would stall every stream on the device while it runs, and a failure in the
// middle of a step is not something the caller can recover from.  The regular backward entry point,
// ab_attn_bwd, needs two scratch buffers from its caller; this variant keeps that scratch inside the
// library instead, in a fixed block of device memory that is part of the loaded module.
//
// ab_attn_bwd_static_scratch computes exactly what ab_attn_bwd computes (dQ, dK, dV of the interval
// masked attention) and takes the same inputs and outputs, minus the two scratch pointers.
//
// Limits and rules
//  * The scratch block is AB_NOALLOC_SCRATCH_BYTES (8 MiB + 64 KiB) per GPU, held by every GPU that
//    loads the library until the process exits.  A call fits when
//        hq * q_total <= AB_NOALLOC_MAX_ROW_STATS   and   ceil(q_total / (128 / (hq / hkv))) <= 4096;
//    otherwise the function launches nothing and returns AB_NOALLOC_TOO_LARGE (-20).
//  * No cudaMalloc, cudaFree or allocating library routine is called, on the first call or later.
//  * The first call on each device looks up the address of the scratch block (once per device, with
//    that device current).  Make that first call before starting any stream capture.
//  * All calls on a device share the one block.  Its contents are whatever the last call left; this
//    kernel overwrites every word it later reads, so nothing has to be cleared between calls.  Two
//    calls that overlap in time on the same GPU (different streams, or different host threads) race
//    on the block: serialise them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define AB_NOALLOC_MAX_ROW_STATS (2 * 1024 * 1024)                       /* floats: hq * q_total */
#define AB_NOALLOC_MAX_QUERY_TILES 4096
#define AB_NOALLOC_SCRATCH_BYTES (AB_NOALLOC_MAX_ROW_STATS * 4 + AB_NOALLOC_MAX_QUERY_TILES * 16)
#define AB_NOALLOC_TOO_LARGE (-20)
#define AB_NOALLOC_SETUP_FAILED (-21)

// q, dout, dq: [q_total, hq, 128] bf16 contiguous.  k, v: [tk, hkv, 128] bf16 with row strides k_ld,
// v_ld (elements).  dk, dv: [tk, hkv, 128] bf16 contiguous.  intervals: [q_total, 4] int32.
// out: forward output, lse: [hq, q_total] fp32 from the forward.  status: device int, set to a
// non-zero code if a bounded wait inside a kernel ran out.  Returns 0 when the kernels were launched.
int ab_attn_bwd_static_scratch(const void* q, const void* k, const void* v, const int* intervals,
                               const void* out, const float* lse, const void* dout, void* dq, void* dk,
                               void* dv, int q_total, int tk, int hq, int hkv, int head_dim,
                               long long k_ld, long long v_ld, float scale, int* status, void* stream);

#ifdef __cplusplus
}
#endif
