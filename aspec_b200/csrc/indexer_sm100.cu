// Lightning-indexer scores and top-k selection for the sparse drafts (DSA / CSA), sm_100a.
//
//   score[q, t] = sum_h  w[q, h] * relu( qi[q, h, :] . ki[t, :] )          t in [lo_q, hi_q)
//
// ab_indexer_scores: a tcgen05 GEMM whose accumulator is transposed on purpose - keys are the M dimension (TMEM
// lanes), the (query, head) pairs of a tile are the N dimension (columns).  The epilogue thread of a key lane then
// owns every head of a query in its own registers: ReLU, the per-head weight and the head sum need no cross-thread
// reduction, and the 128 lanes write 128 consecutive keys of a score row (coalesced).  [n*H, T] logits never exist.
//   warp 0      TMA producer: the tile's 128 (query, head) rows once, then key tiles through a 5-stage ring
//   warp 1      tcgen05.mma issuer, two 128-column accumulators so that the epilogue of tile j runs under tile j+1
//   warps 2..9  epilogue: two warpgroups, each takes half of the accumulator's columns (whole queries when H <= 64), so
//               two warps per scheduler hide each other's tensor-memory load latency
//
// ab_topk_select: one CTA per score row; an 8-bit-per-pass radix select over the order-preserving integer image of
// the floats finds the k-th largest value, then one ordered pass writes the selected key indices in ascending order
// (ties at the threshold go to the lower index).  Rows with at most k eligible keys keep them all; unused slots = -1.
//
// Every mbarrier wait is bounded and reports through the status word.
#include "common.cuh"

namespace ab {
namespace idx {

static constexpr int BM = 128;   // keys per tile
static constexpr int BN = 128;   // (query, head) pairs per tile
static constexpr int kStages = 5;   // 160 KB of key tiles in flight per SM: enough to cover the L2 round trip at one tile per 512 cycles
static constexpr int kThreads = 320;   // TMA warp, MMA warp, two epilogue warpgroups

struct alignas(64) IdxMaps {
  CUtensorMap q, k;
};
struct IdxParams {
  const float* w;     // [n, H]
  const int* lo;      // [n]
  const int* hi;      // [n]
  float* out;         // [n, ld_out]
  long long ld_out;
  int n, T, d_chunks;          // d = 64 * d_chunks
  int key_splits;
  int* status;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
// [rows, d] bf16, row stride `ld` elements; box = 64 columns x 128 rows, 128-byte swizzle, zero fill out of bounds.
static int make_map_2d(CUtensorMap* map, const void* base, long long rows, int d, long long ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    cudaFree(nullptr);   // first device work of this thread: bind the primary context, encode again
    r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : -2;
}

static constexpr int kTileBytes = 128 * 128 * 2;   // 32 KB at d = 128 (two 64-column chunks of 16 KB)
static constexpr int kChunkBytes = 128 * 128;
static constexpr int kSmemBytes = (1 + kStages) * kTileBytes + 1024 /*w, lo, hi*/ + 256 /*barriers*/ + 1024;

template <int H, int kSplit>     // kSplit: epilogue warpgroups that share an accumulator (2 needs H <= 64)
__global__ void __launch_bounds__(kThreads, 1)
indexer_scores_kernel(const __grid_constant__ IdxMaps maps, const IdxParams p) {
  constexpr int NQ = BN / H;   // queries per tile
  constexpr int kCols = BN / kSplit;           // accumulator columns per epilogue thread
  constexpr int NQL = kCols / H;               // queries per epilogue thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  float* sW = reinterpret_cast<float*>(sK + kStages * kTileBytes);   // [128]
  int* sLo = reinterpret_cast<int*>(sW + BN);                        // [NQ]
  int* sHi = sLo + 16;
  int* sRange = sHi + 16;                                            // [2] first / one-past-last key tile of this CTA
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sW) + 1024);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                 // [kStages]
  uint64_t* k_empty = bars + 1 + kStages;      // [kStages]
  uint64_t* acc_full = bars + 1 + 2 * kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;            // [2], 4 arrivals each
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * NQ;
  const int tile_bytes = p.d_chunks * kChunkBytes;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 4 * kSplit); }
    fence_barrier_init();
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    // key tiles any query of this tile can see, cut into this CTA's slice
    int lo = 0x7fffffff, hi = 0;
    for (int i = 0; i < NQ; ++i) {
      const int q = q0 + i;
      const int a = q < p.n ? p.lo[q] : 0, b = q < p.n ? p.hi[q] : 0;
      sLo[i] = a;
      sHi[i] = b;
      if (b > a) { lo = min(lo, a); hi = max(hi, b); }
    }
    if (hi > p.T) hi = p.T;
    int t0 = 0, t1 = 0;
    if (hi > lo) {
      const int first = lo / BM, last = (hi + BM - 1) / BM;
      const int per = (last - first + p.key_splits - 1) / p.key_splits;
      t0 = first + blockIdx.y * per;
      t1 = min(t0 + per, last);
      if (t1 < t0) t1 = t0;
    }
    sRange[0] = t0;
    sRange[1] = t1;
  }
  if (threadIdx.x < BN) {
    const long long gi = (long long)q0 * H + threadIdx.x;
    sW[threadIdx.x] = gi < (long long)p.n * H ? p.w[gi] : 0.f;
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int t0 = sRange[0], t1 = sRange[1];
  const int n_tiles = t1 - t0;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_arrive_expect_tx(q_full, tile_bytes);
      for (int c = 0; c < p.d_chunks; ++c) tma_load_2d(sQ + c * kChunkBytes, &maps.q, q_full, 64 * c, q0 * H);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kStages;
        if (!mbar_wait(&k_empty[st], ((j / kStages) & 1) ^ 1u, abort_word)) break;
        mbar_arrive_expect_tx(&k_full[st], tile_bytes);
        for (int c = 0; c < p.d_chunks; ++c)
          tma_load_2d(sK + st * kTileBytes + c * kChunkBytes, &maps.k, &k_full[st], 64 * c, (t0 + j) * BM);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);   // keys (K-major) x (query, head) rows (K-major)
      const uint32_t q_addr = smem_u32(sQ);
      bool alive = mbar_wait(q_full, 0, abort_word);
      for (int j = 0; j < n_tiles && alive; ++j) {
        const int st = j % kStages, acc = j & 1;
        if (!mbar_wait(&k_full[st], (j / kStages) & 1, abort_word)) break;
        if (!mbar_wait(&acc_empty[acc], ((j >> 1) & 1) ^ 1u, abort_word)) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st * kTileBytes);
        const int ksteps = p.d_chunks * 4;
        for (int k = 0; k < ksteps; ++k) {
          const uint32_t off = (k >> 2) * kChunkBytes + (k & 3) * 32;
          tc_mma_ss(tmem + acc * BN, make_smem_desc(k_addr + off, 16, 1024), make_smem_desc(q_addr + off, 16, 1024),
                    idesc, k ? 1u : 0u);
        }
        tc_commit(&k_empty[st]);
        tc_commit(&acc_full[acc]);
      }
    }
  } else if (((warp - 2) >> 2) < kSplit) {
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int cbeg = half * kCols;
    const uint32_t lane_base = static_cast<uint32_t>(qd * 32) << 16;
    const int r = qd * 32 + lane;            // key row of the tile
    for (int j = 0; j < n_tiles; ++j) {
      const int acc = j & 1;
      if (!mbar_wait(&acc_full[acc], (j >> 1) & 1, abort_word)) break;
      tc_fence_after();
      // four independent partial sums per query: a single chain of H dependent FMAs per tile would take as long as
      // the tile's MMAs
      float part[NQL][4];
#pragma unroll
      for (int i = 0; i < NQL; ++i) part[i][0] = part[i][1] = part[i][2] = part[i][3] = 0.f;
      // all tensor-memory loads of this thread's columns are issued before the one wait: their latencies overlap
      uint32_t s[kCols / 32][32];
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c) tmem_ld_32x32(tmem + lane_base + acc * BN + cbeg + c * 32, s[c]);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < kCols; c += 32) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(sW + cbeg + c + i);   // same address in every lane: broadcast
          float* dst = part[(c + i) / H];
          dst[0] = fmaf(fmaxf(__uint_as_float(s[c / 32][i + 0]), 0.f), w4.x, dst[0]);
          dst[1] = fmaf(fmaxf(__uint_as_float(s[c / 32][i + 1]), 0.f), w4.y, dst[1]);
          dst[2] = fmaf(fmaxf(__uint_as_float(s[c / 32][i + 2]), 0.f), w4.z, dst[2]);
          dst[3] = fmaf(fmaxf(__uint_as_float(s[c / 32][i + 3]), 0.f), w4.w, dst[3]);
        }
      }
      float sum[NQL];
#pragma unroll
      for (int i = 0; i < NQL; ++i) sum[i] = (part[i][0] + part[i][1]) + (part[i][2] + part[i][3]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      const int key = (t0 + j) * BM + r;
      if (key < p.T) {
#pragma unroll
        for (int i = 0; i < NQL; ++i) {
          const int ql = half * NQL + i;
          const int q = q0 + ql;
          if (q < p.n) {
            const bool vis = key >= sLo[ql] && key < sHi[ql];
            p.out[(size_t)q * p.ld_out + key] = vis ? sum[i] : -INFINITY;
          }
        }
      }
    }
  }
  if (*abort_word) {
    __nanosleep(200000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tmem_dealloc(tmem, 256); }
}

template <int H, int SPLIT>
static int launch_scores_v(const IdxMaps& maps, const IdxParams& p, cudaStream_t stream) {
  static std::atomic<unsigned long long> attr_done{0};
  if (!once_per_device(attr_done, [&] {
        return cudaFuncSetAttribute(indexer_scores_kernel<H, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes) == cudaSuccess;
      }))
    return -3;
  const int nq = BN / H;
  const int q_tiles = (p.n + nq - 1) / nq;
  indexer_scores_kernel<H, SPLIT><<<dim3(q_tiles, p.key_splits), kThreads, kSmemBytes, stream>>>(maps, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
// epilogue_groups: 0 = default (two warpgroups when H <= 64), 1 or 2 = forced (benchmarks)
template <int H>
static int launch_scores(const IdxMaps& maps, const IdxParams& p, cudaStream_t stream, int epilogue_groups) {
  if constexpr (H <= 64) {
    if (epilogue_groups != 1) return launch_scores_v<H, 2>(maps, p, stream);
  }
  return launch_scores_v<H, 1>(maps, p, stream);
}

// ------------------------------------------------------------------------------------ top-k ----
__device__ __forceinline__ uint32_t ordered_bits(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float <=> larger unsigned
}

static constexpr int kTopkThreads = 512;

__global__ void __launch_bounds__(kTopkThreads)
topk_select_kernel(const float* __restrict__ scores, long long ld, const int* __restrict__ lo_arr,
                   const int* __restrict__ hi_arr, int T, int k, int* __restrict__ out) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;     // bits decided so far (high bits of the threshold key)
  __shared__ int s_need;            // how many more keys are wanted among those matching the prefix
  __shared__ int warp_tot[2][kTopkThreads / 32];
  const int row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int lo = lo_arr[row], hi = min(hi_arr[row], T);
  if (lo < 0) lo = 0;
  const int count = hi > lo ? hi - lo : 0;
  int* orow = out + (size_t)row * k;
  const float* srow = scores + (size_t)row * ld;
  if (count <= k) {   // keep every eligible key
    for (int i = tid; i < k; i += kTopkThreads) orow[i] = i < count ? lo + i : -1;
    return;
  }
  if (tid == 0) { s_prefix = 0u; s_need = k; }
  __syncthreads();
  // four passes, most significant byte first: after each, the threshold's byte is known
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += kTopkThreads) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < count; i += kTopkThreads) {
      const uint32_t key = ordered_bits(srow[lo + i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need, b = 255;
      for (; b > 0; --b) {          // walk down from the largest byte until the wanted count is covered
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_need = need;                // keys with exactly this prefix still to take
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;    // the k-th largest key; `s_need` of the keys equal to it are taken, lowest index first
  const int need_eq = s_need;
  int gt_base = 0, eq_base = 0;
  for (int i0 = 0; i0 < count; i0 += kTopkThreads) {
    const int i = i0 + tid;
    uint32_t key = 0u;
    const bool in = i < count;
    if (in) key = ordered_bits(srow[lo + i]);
    const bool gt = in && key > thr, eq = in && key == thr;
    const uint32_t bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) { warp_tot[0][warp] = __popc(bg); warp_tot[1][warp] = __popc(be); }
    __syncthreads();
    int gt_before = gt_base + __popc(bg & ((1u << lane) - 1u));
    int eq_before = eq_base + __popc(be & ((1u << lane) - 1u));
    int gt_all = 0, eq_all = 0;
    for (int w = 0; w < kTopkThreads / 32; ++w) {
      if (w < warp) { gt_before += warp_tot[0][w]; eq_before += warp_tot[1][w]; }
      gt_all += warp_tot[0][w];
      eq_all += warp_tot[1][w];
    }
    const bool take = gt || (eq && eq_before < need_eq);
    if (take) {
      const int pos = gt_before + min(eq_before, need_eq);
      if (pos < k) orow[pos] = lo + i;
    }
    gt_base += gt_all;
    eq_base += eq_all;
    __syncthreads();
  }
}

}  // namespace idx
}  // namespace ab

// qi [n, H, d] bf16 contiguous, ki [T, d] bf16 (row stride k_ld elements), w [n, H] fp32, lo / hi [n] int32.
// out [n, ld_out] fp32: every key < T of a key tile that some query of the same query tile can see is written
// (-inf outside the row's own [lo, hi)); other entries are left untouched, so a caller that reads whole rows
// pre-fills `out` with -inf.  H in {8, 16, 32, 64, 128}, d in {64, 128}.
extern "C" int ab_indexer_scores(const void* qi, const void* ki, const float* w, const int* lo, const int* hi, float* out,
                                 long long ld_out, int n, int T, int H, int d, long long k_ld, int epilogue_groups,
                                 int* status, void* stream) {
  using namespace ab;
  using namespace ab::idx;
  if (d != 64 && d != 128) return -10;
  if (n <= 0 || T <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(qi) | reinterpret_cast<uintptr_t>(ki)) & 15) return -12;
  if (k_ld & 7) return -12;
  IdxMaps maps;
  int rc;
  if ((rc = make_map_2d(&maps.q, qi, (long long)n * H, d, d))) return rc;
  if ((rc = make_map_2d(&maps.k, ki, T, d, k_ld))) return rc;
  IdxParams p;
  p.w = w; p.lo = lo; p.hi = hi; p.out = out; p.ld_out = ld_out;
  p.n = n; p.T = T; p.d_chunks = d / 64; p.status = status;
  // few query tiles: cut the key range so that the grid still covers the machine
  const int nq = BN / (H > 0 ? H : 1);
  const int q_tiles = (n + (nq > 0 ? nq : 1) - 1) / (nq > 0 ? nq : 1);
  int splits = 1;
  if (q_tiles < 296) splits = (296 + q_tiles - 1) / q_tiles;
  const int key_tiles = (T + BM - 1) / BM;
  if (splits > key_tiles) splits = key_tiles;
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  p.key_splits = splits;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (H) {
    case 8: return launch_scores<8>(maps, p, s, epilogue_groups);
    case 16: return launch_scores<16>(maps, p, s, epilogue_groups);
    case 32: return launch_scores<32>(maps, p, s, epilogue_groups);
    case 64: return launch_scores<64>(maps, p, s, epilogue_groups);
    case 128: return launch_scores<128>(maps, p, s, epilogue_groups);
    default: return -11;
  }
}

// out [n, k] int32: indices (ascending) of the k largest scores of row r inside [lo[r], hi[r]); -1 pads short rows.
extern "C" int ab_topk_select(const float* scores, long long ld, const int* lo, const int* hi, int n, int T, int k,
                              int* out, void* stream) {
  using namespace ab::idx;
  if (n <= 0 || k <= 0) return 0;
  topk_select_kernel<<<n, kTopkThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(scores, ld, lo, hi, T, k, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
