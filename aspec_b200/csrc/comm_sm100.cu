// Cross-GPU signalling and peer-memory data movement for sm_100a.
//
// Buffers of other GPUs are mapped into this process (CUDA IPC / symmetric memory); kernels here use
// plain ld/st.global on those addresses, which travel over NVLink 5 through the NVSwitch.  No TMA load
// with cluster multicast is used anywhere.  Every wait on a flag that another GPU (or nobody) writes
// is bounded: when the limit runs out the kernel records kStatusPeerTimeout and returns, leaving the
// context usable.
#include "common.cuh"

#include <string.h>

namespace ab {

// flag[0] = value, ordered after every earlier write of this GPU (release at system scope).
__global__ void flag_publish_kernel(long long* flag, long long value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.s64 [%0], %1;" ::"l"(flag), "l"(value) : "memory");
}

// Spin until flag[0] >= value or `limit_ns` passed.  status[0] = kStatusPeerTimeout on expiry.
__global__ void flag_wait_kernel(const long long* flag, long long value, unsigned long long limit_ns,
                                 int* status) {
  const unsigned long long t0 = globaltimer_ns();
  long long seen;
  for (;;) {
    asm volatile("ld.acquire.sys.global.s64 %0, [%1];" : "=l"(seen) : "l"(flag) : "memory");
    if (seen >= value) return;
    if (globaltimer_ns() - t0 > limit_ns) {
      if (status) atomicExch(status, kStatusPeerTimeout);
      return;
    }
    __nanosleep(200);
  }
}

// Copy `n_vec` 16-byte vectors from local memory to a peer mapping (or the reverse) with coalesced
// 128-bit accesses; used for token ids and other small side tensors of a feature slot.
__global__ void copy_vec16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n_vec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

// out[i] = sum over `n_peers` buffers of in_p[i] (bf16 in, bf16 out, fp32 accumulate): the reduce half of
// a reduce-scatter / all-reduce done with peer loads.  Each rank calls it on its own shard range.
struct PeerPtrs {
  const __nv_bfloat16* p[8];
};
__global__ void peer_reduce_bf16_kernel(PeerPtrs peers, int n_peers, __nv_bfloat16* __restrict__ out,
                                        long long n, float scale) {
  const long long nv = n >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < n_peers; ++r) {
      const uint4 u = reinterpret_cast<const uint4*>(peers.p[r])[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0] * scale, acc[1] * scale);
    o.y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
    o.z = pack_bf16x2(acc[4] * scale, acc[5] * scale);
    o.w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

struct PeerPtrsF {
  const float* p[8];
};
// fp32 variant (gradient shards): out = scale * sum_r in_r
__global__ void peer_reduce_f32_kernel(PeerPtrsF peers, int n_peers, float* __restrict__ out, long long n,
                                       float scale) {
  const long long nv = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (int r = 0; r < n_peers; ++r) {
      const float4 v = reinterpret_cast<const float4*>(peers.p[r])[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(out)[i] = acc;
  }
}


// ---- sharded optimizer over peer memory ("reduce-scatter + norm" and "AdamW + all-gather" without a library
// collective).  Every rank owns the element range [lo, lo + n) of the flat parameter space.
//
// Phase 1: shard[i] = sum_r peer_grad[r][lo + i]   (p loads over NVLink, one local store) and the shard's
//          sum of squares / non-finite flag go to ctrl[0] / ctrl[1] (block-reduced, one atomic per block).
__global__ void shard_reduce_sumsq_kernel(PeerPtrsF peers, int n_peers, long long lo, float* __restrict__ shard,
                                          long long n, float* __restrict__ ctrl) {
  float ss = 0.f;
  int bad = 0;
  const long long nv = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (int r = 0; r < n_peers; ++r) {
      const float4 v = *reinterpret_cast<const float4*>(peers.p[r] + lo + 4 * i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(shard)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    bad |= !(isfinite(acc.x) && isfinite(acc.y) && isfinite(acc.z) && isfinite(acc.w));
  }
  __shared__ float red[32];
  __shared__ int red_bad;
  if (threadIdx.x == 0) red_bad = 0;
  __syncthreads();
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  if (bad) atomicOr(&red_bad, 1);
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) {
      atomicAdd(&ctrl[0], v);
      if (red_bad) atomicAdd(&ctrl[1], 1.f);
    }
  }
}

// ---- flags between ranks, for protocols that never call a library collective.  Every rank owns an array
// flags[slot * world + writer]; rank w publishes into element (slot, w) of EVERY rank's array, and a rank waits until
// all `world` elements of one of its own slots reach a value.  Values only grow, so a late waiter still passes.
struct PeerFlagPtrs {
  long long* p[8];
};
__global__ void flags_signal_kernel(PeerFlagPtrs flags, int n_peers, long long index, long long value) {
  if (threadIdx.x < n_peers) {
    __threadfence_system();          // everything this GPU wrote before the launch is visible before the flag
    asm volatile("st.release.sys.global.s64 [%0], %1;" ::"l"(flags.p[threadIdx.x] + index), "l"(value) : "memory");
  }
}
// One thread per flag; bounded like flag_wait_kernel.  status[0] = kStatusPeerTimeout when any flag stayed low.
__global__ void flags_wait_all_kernel(const long long* flags, int count, long long value, unsigned long long limit_ns,
                                      int* status) {
  if (threadIdx.x >= count) return;
  const unsigned long long t0 = globaltimer_ns();
  long long seen;
  for (;;) {
    asm volatile("ld.acquire.sys.global.s64 %0, [%1];" : "=l"(seen) : "l"(flags + threadIdx.x) : "memory");
    if (seen >= value) return;
    if (globaltimer_ns() - t0 > limit_ns) {
      if (status) atomicExch(status, kStatusPeerTimeout);
      return;
    }
    __nanosleep(200);
  }
}

// Parameter all-gather by peer loads: dst[r * shard_vec + i] = shard_r[i] (16-byte vectors); block y = source rank.
struct PeerPtrsV {
  const uint4* p[8];
};
__global__ void peer_gather_kernel(PeerPtrsV shards, long long shard_vec, uint4* __restrict__ dst) {
  const uint4* __restrict__ src = shards.p[blockIdx.y];
  uint4* out = dst + (long long)blockIdx.y * shard_vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < shard_vec;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = src[i];
}

// Gradient reduce-scatter by peer loads, accumulating: shard[i] += sum_r peer_grad[r][lo + i].
__global__ void shard_reduce_accum_kernel(PeerPtrsF peers, int n_peers, long long lo, float* __restrict__ shard,
                                          long long n) {
  const long long nv = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<float4*>(shard)[i];
    for (int r = 0; r < n_peers; ++r) {
      const float4 v = *reinterpret_cast<const float4*>(peers.p[r] + lo + 4 * i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(shard)[i] = acc;
  }
}

struct PeerPtrsW {
  __nv_bfloat16* p[8];
};
// Phase 2: AdamW on the owned shard (fp32 master / moments are shard-sized) and the new bf16 weights stored into
//          EVERY rank's replica of the flat parameter buffer - the parameter all-gather is the epilogue's store.
//          ctrl as in the replicated optimizer: [0] global sum of squares, [1] non-finite flag, [2] pre-scale.
__global__ void shard_adamw_scatter_kernel(float* __restrict__ master, const float* __restrict__ grad,
                                           float* __restrict__ m, float* __restrict__ v, PeerPtrsW params,
                                           int n_peers, long long lo, long long n, const float* __restrict__ ctrl,
                                           float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                           float bc2, float max_norm) {
  if (ctrl[1] > 0.f || !isfinite(ctrl[0])) return;
  if (bc1 <= 0.f) {   // device-side step counter: ctrl[4] = applied updates including this one
    const float t = fmaxf(ctrl[4], 1.f);
    bc1 = 1.f - powf(beta1, t);
    bc2 = 1.f - powf(beta2, t);
  }
  const float pre = ctrl[2];
  const float norm = pre * sqrtf(ctrl[0]);
  float coef = pre;
  if (max_norm > 0.f) coef *= fminf(1.f, max_norm / (norm + 1e-6f));
  const long long nv = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 w4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    const float g[4] = {g4.x * coef, g4.y * coef, g4.z * coef, g4.w * coef};
    float w[4] = {w4.x, w4.y, w4.z, w4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mm[j] = beta1 * mm[j] + (1.f - beta1) * g[j];
      vv[j] = beta2 * vv[j] + (1.f - beta2) * g[j] * g[j];
      w[j] = w[j] * (1.f - lr * wd) - lr * (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    uint2 packed;
    packed.x = pack_bf16x2(w[0], w[1]);
    packed.y = pack_bf16x2(w[2], w[3]);
    for (int r = 0; r < n_peers; ++r) *reinterpret_cast<uint2*>(params.p[r] + lo + 4 * i) = packed;
  }
}

// ---- merge of attention partials over disjoint key sets (direct context parallelism) -------------------------
// One warp per (query row, head): lse = log sum_r exp(lse_r), out = sum_r exp(lse_r - lse) * O_r.  Parts whose lse is
// not finite saw no key for the row; a row that no part saw gets zeros and `empty_lse`.
__global__ void attn_merge_partials_kernel(const __nv_bfloat16* __restrict__ part_o, long long part_stride_o,
                                           const float* __restrict__ part_lse, long long part_stride_lse, int n_parts,
                                           int n_rows, int heads, int head_dim, __nv_bfloat16* __restrict__ out,
                                           float* __restrict__ lse_out, float empty_lse) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)n_rows * heads) return;
  const int row = (int)(warp / heads), h = (int)(warp - (long long)row * heads);
  float l[8], m = -INFINITY;
  for (int r = 0; r < n_parts; ++r) {
    l[r] = part_lse[r * part_stride_lse + (long long)h * n_rows + row];
    if (isfinite(l[r])) m = fmaxf(m, l[r]);
  }
  const bool any = m > -INFINITY;
  float s = 0.f;
  for (int r = 0; r < n_parts; ++r)
    if (any && isfinite(l[r])) s += __expf(l[r] - m);
  const float lse = any ? m + __logf(s) : empty_lse;
  const long long base = ((long long)row * heads + h) * head_dim;
  for (int e = lane * 4; e < head_dim; e += 128) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < n_parts; ++r) {
      if (!any || !isfinite(l[r])) continue;
      const float w = __expf(l[r] - lse);
      const uint2 raw = *reinterpret_cast<const uint2*>(part_o + r * part_stride_o + base + e);
      const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(v[0]), b = __bfloat1622float2(v[1]);
      acc[0] += w * a.x;
      acc[1] += w * a.y;
      acc[2] += w * b.x;
      acc[3] += w * b.y;
    }
    __nv_bfloat162 o[2] = {__floats2bfloat162_rn(acc[0], acc[1]), __floats2bfloat162_rn(acc[2], acc[3])};
    *reinterpret_cast<uint2*>(out + base + e) = *reinterpret_cast<uint2*>(o);
  }
  if (lane == 0) lse_out[(long long)h * n_rows + row] = lse;
}

// ---- vocabulary-parallel merges over peer memory -----------------------------------------------------------
// out[i] = log sum_r exp(lse_r[i])   (each rank's partial log-sum-exp over its vocabulary shard)
__global__ void peer_lse_merge_kernel(PeerPtrsF peers, int n_peers, float* __restrict__ out, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    float m = -INFINITY;
    for (int r = 0; r < n_peers; ++r) {
      v[r] = peers.p[r][i];
      m = fmaxf(m, v[r]);
    }
    float s = 0.f;
    for (int r = 0; r < n_peers; ++r)
      if (v[r] > -INFINITY) s += __expf(v[r] - m);
    out[i] = m + __logf(s);
  }
}
struct PeerPtrsI {
  const int* p[8];
};
// Per row: the arg-max over all shards (largest value, smallest global column on ties) compared with the label.
__global__ void peer_argmax_merge_kernel(PeerPtrsF vals, PeerPtrsI idxs, int n_peers, const long long* __restrict__ labels,
                                         float* __restrict__ correct, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int r = 0; r < n_peers; ++r) {
      const float v = vals.p[r][i];
      const int a = idxs.p[r][i];
      if (v > best || (v == best && a < arg)) {
        best = v;
        arg = a;
      }
    }
    correct[i] = (long long)arg == labels[i] ? 1.f : 0.f;
  }
}

}  // namespace ab

extern "C" {
using namespace ab;

int ab_flag_publish(long long* flag, long long value, void* stream) {
  flag_publish_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_flag_wait(const long long* flag, long long value, double limit_ms, int* status, void* stream) {
  if (limit_ms <= 0 || limit_ms > 10000.0) return -10;   // waits are always bounded (<= 10 s)
  flag_wait_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      flag, value, static_cast<unsigned long long>(limit_ms * 1e6), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_copy_bytes(const void* src, void* dst, long long n_bytes, void* stream) {
  if (n_bytes <= 0) return 0;
  if ((n_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -10;
  const long long nv = n_bytes >> 4;
  long long grid = (nv + 255) / 256;
  if (grid > 148 * 4) grid = 148 * 4;
  copy_vec16_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), nv);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_peer_reduce(const void* const* peer_ptrs, int n_peers, void* out, long long n, float scale, int is_fp32,
                   void* stream) {
  if (n_peers < 1 || n_peers > 8 || n <= 0) return -10;
  long long grid = ((n >> 3) + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid < 1) grid = 1;
  if (is_fp32) {
    if (n & 3) return -10;
    PeerPtrsF pp;
    for (int i = 0; i < n_peers; ++i) pp.p[i] = reinterpret_cast<const float*>(peer_ptrs[i]);
    peer_reduce_f32_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        pp, n_peers, reinterpret_cast<float*>(out), n, scale);
  } else {
    if (n & 7) return -10;
    PeerPtrs pp;
    for (int i = 0; i < n_peers; ++i) pp.p[i] = reinterpret_cast<const __nv_bfloat16*>(peer_ptrs[i]);
    peer_reduce_bf16_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        pp, n_peers, reinterpret_cast<__nv_bfloat16*>(out), n, scale);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Shard element ranges must start and end on multiples of 4 elements (16-byte fp32 vectors, 8-byte bf16 stores).
int ab_shard_reduce_sumsq(const void* const* peer_grads, int n_peers, long long lo, float* shard, long long n,
                          float* ctrl, void* stream) {
  if (n_peers < 1 || n_peers > 8 || n < 0 || (n & 3) || (lo & 3)) return -10;
  if (n == 0) return 0;
  PeerPtrsF pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = reinterpret_cast<const float*>(peer_grads[i]);
  long long grid = ((n >> 2) + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  shard_reduce_sumsq_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pp, n_peers, lo, shard, n, ctrl);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_shard_adamw_scatter(float* master, const float* grad, float* m, float* v, void* const* peer_params, int n_peers,
                           long long lo, long long n, const float* ctrl, float lr, float beta1, float beta2, float eps,
                           float wd, float bc1, float bc2, float max_norm, void* stream) {
  if (n_peers < 1 || n_peers > 8 || n < 0 || (n & 3) || (lo & 3)) return -10;
  if (n == 0) return 0;
  PeerPtrsW pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = reinterpret_cast<__nv_bfloat16*>(peer_params[i]);
  long long grid = ((n >> 2) + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  shard_adamw_scatter_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, grad, m, v, pp, n_peers, lo, n, ctrl, lr, beta1, beta2, eps, wd, bc1, bc2, max_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int ab_flags_signal(void* const* peer_flags, int n_peers, long long index, long long value, void* stream) {
  if (n_peers < 1 || n_peers > 8 || index < 0) return -10;
  PeerFlagPtrs pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = reinterpret_cast<long long*>(peer_flags[i]);
  flags_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pp, n_peers, index, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_flags_wait_all(const long long* flags, int count, long long value, double limit_ms, int* status, void* stream) {
  if (limit_ms <= 0 || limit_ms > 10000.0 || count < 1 || count > 32) return -10;   // waits are always bounded (<= 10 s)
  flags_wait_all_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      flags, count, value, static_cast<unsigned long long>(limit_ms * 1e6), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_peer_gather(const void* const* peer_shards, int n_peers, long long shard_bytes, void* dst, void* stream) {
  if (n_peers < 1 || n_peers > 8 || shard_bytes < 0 || (shard_bytes & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -10;
  if (shard_bytes == 0) return 0;
  PeerPtrsV pp;
  for (int i = 0; i < n_peers; ++i) {
    if (reinterpret_cast<uintptr_t>(peer_shards[i]) & 15) return -10;
    pp.p[i] = reinterpret_cast<const uint4*>(peer_shards[i]);
  }
  const long long nv = shard_bytes >> 4;
  long long gx = (nv + 255) / 256;
  const long long cap = (148 * 8 + n_peers - 1) / n_peers;
  if (gx > cap) gx = cap;
  peer_gather_kernel<<<dim3((unsigned)gx, (unsigned)n_peers), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, nv, reinterpret_cast<uint4*>(dst));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_shard_reduce_accum(const void* const* peer_grads, int n_peers, long long lo, float* shard, long long n,
                          void* stream) {
  if (n_peers < 1 || n_peers > 8 || n < 0 || (n & 3) || (lo & 3)) return -10;
  if (n == 0) return 0;
  PeerPtrsF pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = reinterpret_cast<const float*>(peer_grads[i]);
  long long grid = ((n >> 2) + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  shard_reduce_accum_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pp, n_peers, lo, shard, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int ab_peer_lse_merge(const void* const* peer_lse, int n_peers, float* out, long long n, void* stream) {
  if (n_peers < 1 || n_peers > 8 || n <= 0) return n == 0 ? 0 : -10;
  PeerPtrsF pp;
  for (int i = 0; i < n_peers; ++i) pp.p[i] = reinterpret_cast<const float*>(peer_lse[i]);
  long long grid = (n + 255) / 256;
  if (grid > 148 * 4) grid = 148 * 4;
  peer_lse_merge_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pp, n_peers, out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
// out[n_rows, heads, head_dim] (bf16) and lse_out[heads, n_rows] from `n_parts` partial results laid out with the
// given strides (elements) between parts.  head_dim must be a multiple of 4 and all row bases 8-byte aligned.
int ab_attn_merge_partials(const void* part_o, long long part_stride_o, const float* part_lse, long long part_stride_lse,
                           int n_parts, int n_rows, int heads, int head_dim, void* out, float* lse_out, float empty_lse,
                           void* stream) {
  if (n_parts < 1 || n_parts > 8 || (head_dim & 3)) return -10;
  if (n_rows <= 0) return 0;
  const long long warps = (long long)n_rows * heads;
  const int block = 256;
  const long long grid = (warps * 32 + block - 1) / block;
  attn_merge_partials_kernel<<<(unsigned)grid, block, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(part_o), part_stride_o, part_lse, part_stride_lse, n_parts, n_rows, heads, head_dim,
      reinterpret_cast<__nv_bfloat16*>(out), lse_out, empty_lse);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int ab_peer_argmax_merge(const void* const* peer_vals, const void* const* peer_idxs, int n_peers, const long long* labels,
                         float* correct, long long n, void* stream) {
  if (n_peers < 1 || n_peers > 8 || n <= 0) return n == 0 ? 0 : -10;
  PeerPtrsF pv;
  PeerPtrsI pi;
  for (int i = 0; i < n_peers; ++i) {
    pv.p[i] = reinterpret_cast<const float*>(peer_vals[i]);
    pi.p[i] = reinterpret_cast<const int*>(peer_idxs[i]);
  }
  long long grid = (n + 255) / 256;
  if (grid > 148 * 4) grid = 148 * 4;
  peer_argmax_merge_kernel<<<(int)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pv, pi, n_peers, labels, correct, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
}  // extern "C"

// Lets kernels running on `local` dereference memory of `peer` (both GPUs of this node).  IPC-mapped or
// cudaMalloc'ed peer memory is only reachable from a kernel once the local context enabled peer access.
// Returns 0 on success or when access was already enabled, -1 when the pair has no peer path.
extern "C" int ab_enable_peer_access(int local, int peer) {
  if (local == peer) return 0;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, local, peer) != cudaSuccess || !can) return -1;
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(local) != cudaSuccess) return -2;
  cudaError_t rc = cudaDeviceEnablePeerAccess(peer, 0);
  if (rc == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();   // clear the sticky-free error state
    rc = cudaSuccess;
  }
  if (prev >= 0) cudaSetDevice(prev);
  return rc == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------- symmetric memory -------------
// Buffers that other processes of this node map and that kernels of other GPUs read or write.
// They are allocated here with cudaMalloc (one allocation = one IPC handle, offset zero) and opened in
// the importing process with the *accessing* device current and lazy peer access, so the mapping is
// created in the context whose kernels will dereference it.
extern "C" int ab_symm_alloc(unsigned long long bytes, void** ptr) {
  if (!ptr || bytes == 0) return -10;
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return -5;
  if (cudaMemset(*ptr, 0, bytes) != cudaSuccess) return -6;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : -7;
}
extern "C" int ab_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int ab_ipc_export(void* ptr, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return -1;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
extern "C" int ab_ipc_import(const unsigned char* handle64, int accessing_device, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(accessing_device) != cudaSuccess) return -2;
  const cudaError_t rc = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (prev >= 0) cudaSetDevice(prev);
  return rc == cudaSuccess ? 0 : -3;
}
extern "C" int ab_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
