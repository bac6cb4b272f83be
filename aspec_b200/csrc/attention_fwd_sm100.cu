// Interval-masked flash attention forward for sm_100a (tcgen05 + TMEM + TMA).
//
//   O[i, h, :] = softmax_k( scale * Q[i, h, :] . K[k, h / G, :] + mask(i, k) ) V[k, h / G, :]
//   mask(i, k) = 0 if k in [a0_i, a1_i) U [b0_i, b1_i), else -inf
//
// One CTA owns 128 query rows of one key/value head.  The G = Hq / Hkv query
// heads that share that key/value head are folded into the row dimension
// (row = position * G + head-in-group), so every K/V tile that is staged in
// shared memory serves all of them.  Value head dimension 128; query/key head dimension 128, or 192 for
// materialised-MLA heads (128 "nope" + 64 rotary dims): the kernel is a template on it, the 192 variant stages three
// 64-column chunks of Q and K and runs one CTA per SM.
//
//   warp 0      TMA producer: Q once, then one K and one V buffer, refilled as soon
//               as the MMA that read them has completed
//   warp 1      tcgen05.mma issuer:  S = Q K^T  (128 x 128 x 128),  O += P V
//   warps 2..5  softmax: one tcgen05.ld pass brings the row's 128 scores into
//               registers; max, exp2 and the row sum run on them; P goes back as bf16
//               into the first 64 columns of the S region (A operand of the PV MMA);
//               O stays in TMEM and is rescaled lazily
//
// Two CTAs are resident per SM (96 KB shared memory, 256 TMEM columns each): while one
// CTA's softmax warps work, the other CTA's MMAs keep the tensor core busy, and two
// warps per scheduler hide each other's dependent-issue latency.  Tiles that every row
// of a warp sees completely take a path without any per-element masking.
//
// TMEM columns: S / P [0,128)   O [128,256)
// Every wait is bounded; a timeout sets status[0] and the CTA drains and exits.
#include "common.cuh"

namespace ab {
namespace attn {

static constexpr int BM = 128;   // query rows per CTA (positions x heads-in-group)
static constexpr int BN = 128;   // keys per tile
static constexpr int HD = 128;   // value head dim (and the query/key head dim of ordinary heads)
static constexpr int kThreads = 192;
static constexpr int kKVBytes = BN * HD * 2;      // 32 KB: the V tile (and the K tile at head dim 128)
static constexpr int kChunk = BM * 128;           // bytes of one 64-column chunk (128 rows x 128 B)
// Q and K tiles are HDQK / 64 chunks each
template <int HDQK> struct FwdSmem {
  static constexpr int kQBytes = BM * HDQK * 2;
  static constexpr int kKBytes = BN * HDQK * 2;
  static constexpr int kBytes = kQBytes + kKBytes + kKVBytes + 1024 + 256;
};
static constexpr uint32_t kColS = 0, kColO = 128, kTmemCols = 256;
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr float kRescaleThreshold = 8.0f;  // log2 domain: lazy rescale when max grows > 2^8
static constexpr uint32_t kNegInf = 0xff800000u;

struct FwdParams {
  const int* intervals;   // [Qtot, 4]
  __nv_bfloat16* out;     // [Qtot, Hq, HD]
  float* lse;             // [Hq, Qtot]  natural log
  int q_total, hq, hkv, group, tk;
  float scale_log2;       // softmax scale * log2(e)
  int* status;
};
struct alignas(64) FwdMaps {
  CUtensorMap q, k, v;
};

template <int HDQK>
__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_kernel(const __grid_constant__ FwdMaps maps, const FwdParams p) {
  constexpr int kQBytes = FwdSmem<HDQK>::kQBytes, kKBytes = FwdSmem<HDQK>::kKBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kQBytes;
  uint8_t* sV = sK + kKBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kKVBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;        // 4 arrivals: one per softmax warp
  uint64_t* o_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* range = reinterpret_cast<int*>(tmem_slot + 2);  // [4] c_lo, c_hi, b_lo, b_hi (tile units)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  const int pm = BM / G;                       // positions per tile
  const int q0 = blockIdx.x * pm;              // first position of the tile
  const int kvh = blockIdx.y;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    fence_barrier_init();
    range[0] = range[2] = 0x7fffffff;
    range[1] = range[3] = 0;
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Row intervals (softmax threads) and the tile ranges of this CTA.
  int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
  int my_pos = -1;
  if (warp >= 2) {
    const int t = (warp & 3) * 32 + lane;      // TMEM lane == tile row
    my_pos = q0 + t / G;
    if (my_pos < p.q_total) {
      const int4 iv = reinterpret_cast<const int4*>(p.intervals)[my_pos];
      a0 = iv.x; a1 = iv.y; b0 = iv.z; b1 = iv.w;
      if (a1 > a0) {
        atomicMin(&range[0], a0 / BN);
        atomicMax(&range[1], (a1 + BN - 1) / BN);
      }
      if (b1 > b0) {
        atomicMin(&range[2], b0 / BN);
        atomicMax(&range[3], (b1 + BN - 1) / BN);
      }
    }
  }
  __syncthreads();
  // Two tile ranges [ca, cb) and [da, db); the second starts after the first when they overlap.
  int ca = range[0], cb = range[1], da = range[2], db = range[3];
  if (cb <= ca) { ca = 0; cb = 0; }
  if (db <= da) { da = 0; db = 0; }
  if (cb > ca && db > da) {
    if (da < ca) {  // keep ascending order: swap so the first range starts lower
      int t0 = ca, t1 = cb; ca = da; cb = db; da = t0; db = t1;
    }
    if (da < cb) da = cb;
    if (db < da) db = da;
  }
  const int n_tiles = (cb - ca) + (db - da);
  auto tile_index = [&](int j) { return j < (cb - ca) ? ca + j : da + (j - (cb - ca)); };

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_arrive_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int c = 0; c < HDQK / 64; ++c) tma_load_3d(sQ + c * kChunk, &maps.q, q_full, 64 * c, kvh * G, q0);
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t ph = j & 1;
        const int k0 = tile_index(j) * BN;
        if (!mbar_wait(k_empty, ph ^ 1u, abort_word)) break;        // S_{j-1} has read the K buffer
        mbar_arrive_expect_tx(k_full, kKBytes);
#pragma unroll
        for (int c = 0; c < HDQK / 64; ++c) tma_load_3d(sK + c * kChunk, &maps.k, k_full, 64 * c, kvh, k0);
        if (!mbar_wait(v_empty, ph ^ 1u, abort_word)) break;        // P_{j-1} V_{j-1} has read the V buffer
        mbar_arrive_expect_tx(v_full, kKVBytes);
        tma_load_3d(sV, &maps.v, v_full, 0, kvh, k0);
        tma_load_3d(sV + kChunk, &maps.v, v_full, 64, kvh, k0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(BM, HD, 0, 1);   // P (TMEM)   x V (MN-major)
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool alive = mbar_wait(q_full, 0, abort_word);
      for (int j = 0; j < n_tiles && alive; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_full, ph, abort_word)) break;
        tc_fence_after();
        // S_j overwrites the region P_{j-1} lives in: the tensor core executes in issue order, so it runs
        // after P_{j-1} V_{j-1} has consumed P.
#pragma unroll
        for (int k = 0; k < HDQK / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunk + (k & 3) * 32;
          tc_mma_ss(tmem + kColS, make_smem_desc(q_addr + off, 16, 1024),
                    make_smem_desc(k_addr + off, 16, 1024), idesc_s, k ? 1u : 0u);
        }
        tc_commit(k_empty);
        tc_commit(s_full);
        if (!mbar_wait(v_full, ph, abort_word)) break;
        if (!mbar_wait(p_full, ph, abort_word)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          // V is MN-major: 64-wide dv chunks are kChunk apart, 16 keys = 2048 B.
          tc_mma_ts(tmem + kColO, tmem + kColS + k * 8, make_smem_desc(v_addr + k * 2048, kChunk, 1024),
                    idesc_o, (j | k) ? 1u : 0u);
        }
        tc_commit(v_empty);
        tc_commit(o_full);
      }
    }
  } else {
    // ------------------------------------------------------- softmax --------
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const float sc = p.scale_log2;
    float m_used = -INFINITY, l_sum = 0.f;
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_word)) { alive = false; break; }
      tc_fence_after();
      const int k0 = tile_index(j) * BN;
      // visible columns of this tile for my row, tile-local: [la, ha) U [lb, hb)
      const int la = max(a0 - k0, 0), ha = min(a1 - k0, BN);
      const int lb = max(b0 - k0, 0), hb = min(b1 - k0, BN);
      const bool none = (ha <= la) && (hb <= lb);
      const bool full = (la == 0 && ha == BN) || (lb == 0 && hb == BN);
      const bool warp_full = __all_sync(0xffffffffu, full);
      const bool warp_none = __all_sync(0xffffffffu, none);
      const uint32_t wa = ha > la ? static_cast<uint32_t>(ha - la) : 0u;
      const uint32_t wb = hb > lb ? static_cast<uint32_t>(hb - lb) : 0u;
      // 64 score columns (two 32-column loads in flight) -> registers; masked unless the whole warp sees the tile
      auto load_half = [&](int h, uint32_t (&r)[2][32]) {
        tmem_ld_32x32(tmem + lane_base + kColS + h * 64, r[0]);
        tmem_ld_32x32(tmem + lane_base + kColS + h * 64 + 32, r[1]);
        tmem_ld_wait();
        if (!warp_full) {
          // branch-free visibility: column c is visible iff (c - la) <u (ha - la) or (c - lb) <u (hb - lb)
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const uint32_t col = static_cast<uint32_t>(h * 64 + c * 32 + i);
              const bool vis = (col - static_cast<uint32_t>(la) < wa) | (col - static_cast<uint32_t>(lb) < wb);
              r[c][i] = vis ? r[c][i] : kNegInf;
            }
        }
      };
      // pass 1: row max, four independent chains
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (!warp_none) {
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t r[2][32];
          load_half(h, r);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            mx[0] = fmaxf(mx[0], __uint_as_float(r[0][i]));
            mx[1] = fmaxf(mx[1], __uint_as_float(r[0][i + 1]));
            mx[2] = fmaxf(mx[2], __uint_as_float(r[1][i]));
            mx[3] = fmaxf(mx[3], __uint_as_float(r[1][i + 1]));
          }
        }
      }
      const float rmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sc;   // scale > 0; -inf stays -inf
      const float m_cand = fmaxf(m_used, rmax);
      const bool need = (m_cand > m_used) && (m_used == -INFINITY || m_cand - m_used > kRescaleThreshold);
      const float alpha = need ? (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_cand)) : 1.f;
      if (need) {
        m_used = m_cand;
        l_sum *= alpha;
      }
      // s_full of tile j implies P_{j-1} V_{j-1} has completed: O may be rescaled now
      if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(tmem + lane_base + kColO + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tmem + lane_base + kColO + c, o);
        }
      }
      // pass 2: P = exp2(s * scale - m) as bf16 pairs over the score columns already consumed
      // (64 scores -> 32 words: half h goes to columns [32 h, 32 h + 32) of the S region)
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;   // a row that has seen no key yet: exp2(-inf) = 0
      float sm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t packed[32];
        if (!warp_none) {
          uint32_t r[2][32];
          load_half(h, r);
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float e0 = fast_exp2(fmaf(__uint_as_float(r[c][i]), sc, neg_m));
              const float e1 = fast_exp2(fmaf(__uint_as_float(r[c][i + 1]), sc, neg_m));
              sm[c * 2 + ((i >> 1) & 1)] += e0 + e1;
              packed[c * 16 + (i >> 1)] = pack_bf16x2(e0, e1);
            }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) packed[i] = 0u;
        }
        tmem_st_32x32(tmem + lane_base + kColS + h * 32, packed);
      }
      l_sum += (sm[0] + sm[1]) + (sm[2] + sm[3]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ------------------------------------------------------- epilogue -------
    if (alive && n_tiles > 0) alive = mbar_wait(o_full, (n_tiles - 1) & 1, abort_word);
    if (alive) {
      tc_fence_after();
      const int t = q * 32 + lane;
      const bool row_ok = my_pos >= 0 && my_pos < p.q_total;
      const int head = kvh * G + t % G;
      const float inv = (l_sum > 0.f) ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)(row_ok ? my_pos : 0) * p.hq + head) * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem + lane_base + kColO + c, o);
          tmem_ld_wait();
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            if (n_tiles > 0 && l_sum > 0.f) {
              w.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            } else {
              w = make_uint4(0, 0, 0, 0);
            }
            reinterpret_cast<uint4*>(orow + c)[i] = w;
          }
        }
      }
      if (row_ok)
        p.lse[(size_t)head * p.q_total + my_pos] =
            (l_sum > 0.f) ? (m_used + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
    }
  }

  if (*abort_word) {
    __nanosleep(200000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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

// [rows, heads, hd] bf16 with row stride `ld` elements; box = 64 x box_heads x box_rows.
int make_map_rows_heads_d(CUtensorMap* map, const void* base, long long rows, int heads, long long ld,
                          int box_heads, int box_rows, int hd) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)ld * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // first device work of this thread: bind the primary context of the operand's device and encode again
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, base) == cudaSuccess && at.device >= 0) cudaSetDevice(at.device);
    cudaFree(nullptr);
    r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : -2;
}
int make_map_rows_heads(CUtensorMap* map, const void* base, long long rows, int heads, long long ld,
                        int box_heads, int box_rows) {
  return make_map_rows_heads_d(map, base, rows, heads, ld, box_heads, box_rows, HD);
}

template <int HDQK>
static int launch_fwd(const FwdMaps& maps, const FwdParams& p, dim3 grid, cudaStream_t stream) {
  static std::atomic<unsigned long long> attr_done{0};
  if (!once_per_device(attr_done, [&] {
        return cudaFuncSetAttribute(attn_fwd_kernel<HDQK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    FwdSmem<HDQK>::kBytes) == cudaSuccess;
      }))
    return -3;
  attn_fwd_kernel<HDQK><<<grid, kThreads, FwdSmem<HDQK>::kBytes, stream>>>(maps, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace attn
}  // namespace ab

// `head_dim` is the query/key head dimension: 128, or 192 for materialised-MLA heads; values and the output are
// always 128 wide.  q [Qtot, Hq, head_dim] contiguous; k [Tk, Hkv, head_dim] / v [Tk, Hkv, 128] with row strides.
extern "C" int ab_attn_fwd(const void* q, const void* k, const void* v, const int* intervals, void* out,
                           float* lse, int q_total, int tk, int hq, int hkv, int head_dim,
                           long long k_ld, long long v_ld, float scale, int* status, void* stream) {
  using namespace ab;
  using namespace ab::attn;
  if ((head_dim != HD && head_dim != 192) || hq % hkv) return -10;
  const int G = hq / hkv;
  if (G > 16 || (BM % G)) return -11;
  if (q_total <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return -12;
  if ((k_ld & 7) || (v_ld & 7)) return -12;
  FwdMaps maps;
  const int pm = BM / G;
  int rc;
  if ((rc = make_map_rows_heads_d(&maps.q, q, q_total, hq, (long long)hq * head_dim, G, pm, head_dim))) return rc;
  if ((rc = make_map_rows_heads_d(&maps.k, k, tk, hkv, k_ld, 1, BN, head_dim))) return rc;
  if ((rc = make_map_rows_heads(&maps.v, v, tk, hkv, v_ld, 1, BN))) return rc;
  FwdParams p;
  p.intervals = intervals;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.q_total = q_total;
  p.hq = hq;
  p.hkv = hkv;
  p.group = G;
  p.tk = tk;
  p.scale_log2 = scale * kLog2e;
  p.status = status;
  dim3 grid((q_total + pm - 1) / pm, hkv);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return head_dim == HD ? launch_fwd<128>(maps, p, grid, s) : launch_fwd<192>(maps, p, grid, s);
}
