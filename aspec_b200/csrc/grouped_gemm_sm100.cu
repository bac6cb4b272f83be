// Grouped bf16 GEMM for sm_100a: one persistent launch over a table of output tiles that belong to
// different problems (experts of a mixture-of-experts layer, possibly with operands in several
// GPUs' memories).
//
//   for every tile t:   D_t[rows_t, cols_t] = sum over segments g of t   A_g[128, 64 * kb_g] * B_g[256, 64 * kb_g]^T
//
// A tile names its destination (pointer of its first element, leading dimension, how many rows and
// columns of the 128 x 256 block are stored) and a run of K segments.  A segment names the tensor map
// and the coordinates of its A and B slabs and how many 64-wide k-blocks it spans.  That covers
//   * the expert forward and input-gradient GEMMs (one segment per tile; the A rows of an expert are a
//     slice of a token buffer that may live in a peer GPU's memory, B is a slice of the stacked weights),
//   * the expert weight-gradient GEMMs (the reduction runs over token rows: one segment per source
//     buffer, so the gradients of one expert with tokens from several ranks accumulate in TMEM),
// with the same pipeline as the dense kernel: TMA into 128-byte-swizzled shared memory, tcgen05.mma
// issued by one thread, two 256-column TMEM accumulators, four epilogue warps.
//
// Rows of a slab beyond the problem's own rows are whatever follows in memory (or the TMA zero fill past
// the end of the tensor).  For row-indexed outputs they are masked at the store.  For reductions over
// rows the caller pads one of the two operands with zero rows up to the next multiple of 64 and keeps
// the other operand finite.
//
// The reference runs a Python loop over experts with one cuBLAS GEMM each
// (aspec/models/draft/ling_moe.py:101-115); there is no grouped kernel in it.
#include <cstdio>
#include <cstdlib>
#include "common.cuh"

namespace abg {

using namespace ab;

static constexpr int BM = 128;
static constexpr int BN = 256;
static constexpr int BK = 64;
static constexpr int UMMA_K = 16;
static constexpr int kStages = 4;
static constexpr int kAccBufs = 2;
static constexpr int kTmemCols = 512;
static constexpr int kThreads = 192;  // warp0 TMA, warp1 MMA, warps 2..5 epilogue
static constexpr int kATileBytes = BM * BK * 2;
static constexpr int kBTileBytes = BN * BK * 2;
static constexpr int kStageBytes = kATileBytes + kBTileBytes;
static constexpr int kStoreStageBytes = 4 * 32 * 256;  // per epilogue warp: 32 rows x 128 bf16 columns
static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kStoreStageBytes;
static constexpr int kMaxMaps = 12;

struct alignas(16) GTile {
  void* d;          // first element of the tile in the destination
  long long ldd;    // elements
  int rows, cols;   // stored extent (<= 128, <= 256)
  int seg0, nseg;   // segments [seg0, seg0 + nseg)
};
struct alignas(16) GSeg {
  int a_map, a_mn, a_k;   // tensor map index, coordinate of the tile's first row (or column when MN-major), first k
  int b_map, b_mn, b_k;
  int k_blocks, pad;
};
static_assert(sizeof(GTile) == 32 && sizeof(GSeg) == 32, "table layout is shared with the host");

struct alignas(64) GMaps {
  CUtensorMap m[kMaxMaps];
};

struct GParams {
  const GTile* tiles;
  const GSeg* segs;
  int n_tiles;
  int d_is_fp32;
  float alpha;
  int* status;
};

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GMaps maps, const GParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_empty = bars + 2 * kStages + kAccBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAccBufs);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer ---------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int t = blockIdx.x; alive && t < p.n_tiles; t += gridDim.x) {
        const GTile tile = p.tiles[t];
        for (int g = tile.seg0; alive && g < tile.seg0 + tile.nseg; ++g) {
          const GSeg sg = p.segs[g];
          const CUtensorMap* ma = &maps.m[sg.a_map];
          const CUtensorMap* mb = &maps.m[sg.b_map];
          for (int kb = 0; kb < sg.k_blocks; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word)) { alive = false; break; }
            uint8_t* sa = smem + stage * kStageBytes;
            uint8_t* sb = sa + kATileBytes;
            mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_2d(sa + j * (BK * 128), ma, &full_bar[stage], sg.a_mn + j * 64, sg.a_k + kb * BK);
            } else {
              tma_load_2d(sa, ma, &full_bar[stage], sg.a_k + kb * BK, sg.a_mn);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (BK * 128), mb, &full_bar[stage], sg.b_mn + j * 64, sg.b_k + kb * BK);
            } else {
              tma_load_2d(sb, mb, &full_bar[stage], sg.b_k + kb * BK, sg.b_mn);
            }
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer -----------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      for (int t = blockIdx.x; alive && t < p.n_tiles; t += gridDim.x) {
        const GTile tile = p.tiles[t];
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_word)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        bool first = true;
        for (int g = tile.seg0; alive && g < tile.seg0 + tile.nseg; ++g) {
          const int k_blocks = p.segs[g].k_blocks;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase, abort_word)) { alive = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * kStageBytes);
            const uint32_t sb = sa + kATileBytes;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                       : make_smem_desc(sa + k * 32, 16, 1024);
              const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                       : make_smem_desc(sb + k * 32, 16, 1024);
              tc_mma_ss(d_tmem, da, db, idesc, (first && k == 0) ? 0u : 1u);
            }
            first = false;
            tc_commit(&empty_bar[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
        if (alive) tc_commit(&acc_full[acc]);
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------ epilogue warps -------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const float alpha = p.alpha;
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
      const GTile tile = p.tiles[t];
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_word)) break;
      tc_fence_after();
      const int row = q * 32 + lane;
      const bool row_ok = row < tile.rows;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
      // a tile without segments (an expert that received no rows) stores zeros
      const bool has = tile.nseg > 0;
      auto val = [&](uint32_t bits) { return has ? __uint_as_float(bits) * alpha : 0.f; };
      // Full-width bf16 tiles (the destination may be a peer GPU's memory) are transposed through shared memory so that
      // each store instruction writes two whole 256-byte row segments.
      const bool staged = !p.d_is_fp32 && tile.cols == BN && (tile.ldd & 7) == 0 &&
                          (reinterpret_cast<uintptr_t>(tile.d) & 15) == 0;
      if (staged) {
        uint8_t* stg = smem + kStages * kStageBytes + 256 + q * (32 * 256);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + half * 128 + cc * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o;
              o.x = pack_bf16x2(val(r[8 * i]), val(r[8 * i + 1]));
              o.y = pack_bf16x2(val(r[8 * i + 2]), val(r[8 * i + 3]));
              o.z = pack_bf16x2(val(r[8 * i + 4]), val(r[8 * i + 5]));
              o.w = pack_bf16x2(val(r[8 * i + 6]), val(r[8 * i + 7]));
              const int chunk = cc * 4 + i;
              *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
            }
          }
          __syncwarp();
#pragma unroll 1
          for (int r2 = 0; r2 < 16; ++r2) {
            const int rr = 2 * r2 + (lane >> 4);
            const int ch = lane & 15;
            const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((ch ^ (rr & 15)) << 4));
            const int trow = q * 32 + rr;
            if (trow < tile.rows)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(tile.d) + (long long)trow * tile.ldd +
                                        half * 128 + ch * 8) = o;
          }
          __syncwarp();
        }
      }
#pragma unroll 1
      for (int c = staged ? BN : 0; c < BN; c += 32) {
        const int ncol = tile.cols - c;
        if (ncol <= 0) break;               // uniform over the CTA
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (p.d_is_fp32) {
          float* drow = reinterpret_cast<float*>(tile.d) + (long long)row * tile.ldd + c;
          if (ncol >= 32 && (tile.ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(drow) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(drow)[i] =
                  make_float4(val(r[4 * i]), val(r[4 * i + 1]), val(r[4 * i + 2]), val(r[4 * i + 3]));
          } else {
            for (int i = 0; i < 32 && i < ncol; ++i) drow[i] = val(r[i]);
          }
        } else {
          __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(tile.d) + (long long)row * tile.ldd + c;
          if (ncol >= 32 && (tile.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(drow) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o;
              o.x = pack_bf16x2(val(r[8 * i]), val(r[8 * i + 1]));
              o.y = pack_bf16x2(val(r[8 * i + 2]), val(r[8 * i + 3]));
              o.z = pack_bf16x2(val(r[8 * i + 4]), val(r[8 * i + 5]));
              o.w = pack_bf16x2(val(r[8 * i + 6]), val(r[8 * i + 7]));
              reinterpret_cast<uint4*>(drow)[i] = o;
            }
          } else {
            for (int i = 0; i < 32 && i < ncol; ++i) drow[i] = __float2bfloat16(val(r[i]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------------------------- teardown -----
  if (*abort_word) {
    __nanosleep(200000);  // copies already issued land before the shared memory goes away
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host ----
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

static int encode(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_cols,
                  int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  auto call = [&]() {
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = call();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a thread without a current context (an autograd worker): bind the operand's device and encode again
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, base) == cudaSuccess && at.device >= 0) cudaSetDevice(at.device);
    cudaFree(nullptr);
    r = call();
  }
  if (r != CUDA_SUCCESS && getenv("AB_DEBUG"))
    fprintf(stderr, "grouped gemm: cuTensorMapEncodeTiled failed: CUresult %d base %p rows %lld cols %lld ld %lld\n",
            (int)r, base, rows, cols, ld);
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <int A_MN, int B_MN>
static int launch(const GMaps& maps, const GParams& p, int max_ctas, cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<A_MN, B_MN>;
  static std::atomic<unsigned long long> attr_done{0};   // one per template instantiation, one bit per device
  if (!once_per_device(attr_done, [&] {
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess;
      }))
    return -3;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = p.n_tiles;
  const int cap = max_ctas > 0 ? max_ctas : sms;
  if (grid > cap) grid = cap;
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, kSmemBytes, stream>>>(maps, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace abg

// One bf16 matrix as stored in memory.  role 0: A operand, 1: B operand.  mn_major as in the dense GEMM.
struct AbGroupedOperand {
  const void* ptr;
  long long rows, cols, ld;   // extent of the whole buffer as stored (rows x cols, leading dimension in elements)
  int role;
  int mn_major;
};

extern "C" {

// tiles / segs: device arrays of abg::GTile / abg::GSeg (32 bytes each, layout in the header comment of the
// kernel).  Every operand of a launch shares the A / B majorness given here.  Returns 0 on a successful launch.
int ab_grouped_gemm_bf16(int n_maps, const AbGroupedOperand* ops, const void* tiles, int n_tiles, const void* segs,
                         int a_mn, int b_mn, int d_is_fp32, float alpha, int* status, int max_ctas, void* stream) {
  using namespace abg;
  if (n_maps <= 0 || n_maps > kMaxMaps || n_tiles < 0) return -10;
  if (n_tiles == 0) return 0;
  GMaps maps;
  for (int i = 0; i < n_maps; ++i) {
    const AbGroupedOperand& o = ops[i];
    if ((reinterpret_cast<uintptr_t>(o.ptr) & 15) || (o.ld & 7)) return -12;
    const int mn = o.role == 0 ? a_mn : b_mn;
    if (o.mn_major != mn) return -11;
    int rc;
    if (mn)
      rc = encode(&maps.m[i], o.ptr, o.rows, o.cols, o.ld, 64, BK);          // stored [K, MN]: 64 (mn) x 64 (k)
    else
      rc = encode(&maps.m[i], o.ptr, o.rows, o.cols, o.ld, BK, o.role == 0 ? BM : BN);
    if (rc) return rc;
  }
  for (int i = n_maps; i < kMaxMaps; ++i) maps.m[i] = maps.m[0];
  GParams p;
  p.tiles = reinterpret_cast<const GTile*>(tiles);
  p.segs = reinterpret_cast<const GSeg*>(segs);
  p.n_tiles = n_tiles;
  p.d_is_fp32 = d_is_fp32;
  p.alpha = alpha;
  p.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch<0, 0>(maps, p, max_ctas, s);
  if (!a_mn && b_mn) return launch<0, 1>(maps, p, max_ctas, s);
  if (a_mn && !b_mn) return launch<1, 0>(maps, p, max_ctas, s);
  return launch<1, 1>(maps, p, max_ctas, s);
}

}  // extern "C"
