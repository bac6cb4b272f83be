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
