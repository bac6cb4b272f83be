// Interval-masked flash attention forward for sm_100a (tcgen05 + TMEM + TMA).
//
//   O[i, h, :] = softmax_k( scale * Q[i, h, :] . K[k, h / G, :] + mask(i, k) ) V[k, h / G, :]
//   mask(i, k) = 0 if k in [a0_i, a1_i) U [b0_i, b1_i), else -inf
//
// One CTA owns 128 query rows of one key/value head.  The G = Hq / Hkv query
// heads that share that key/value head are folded into the row dimension
// (row = position * G + head-in-group), so every K/V tile that is staged in
// shared memory serves all of them.  Head dimension 128 (qk and v).
//
//   warp 0      TMA producer: Q once, then K/V tiles (2 stages)
//   warp 1      tcgen05.mma issuer:  S = Q K^T  (128 x 128 x 128),  O += P V
//   warps 2..5  softmax: tcgen05.ld S -> mask -> online softmax (exp2 domain)
//               -> P as bf16 back into TMEM (A operand of the PV MMA), and the
//               conditional rescale of the O accumulator, which stays in TMEM
//
// S_{j+1} is issued before P_j V_j so the softmax of tile j+1 overlaps the PV
// MMA of tile j; P is double-buffered for the same reason.
//
// TMEM columns: S [0,128)  O [128,256)  P0 [256,320)  P1 [320,384)   (512 allocated)
// Every wait is bounded; a timeout sets status[0] and the CTA drains and exits.
#include "common.cuh"

namespace ab {
namespace attn {

static constexpr int BM = 128;   // query rows per CTA (positions x heads-in-group)
static constexpr int BN = 128;   // keys per tile
static constexpr int HD = 128;   // head dim
static constexpr int kStages = 2;
static constexpr int kThreads = 192;
static constexpr int kQBytes = BM * HD * 2;       // 32 KB (two 64-column swizzled chunks)
static constexpr int kKVBytes = BN * HD * 2;      // 32 KB each for K and V
static constexpr int kChunk = BM * 128;           // bytes of one 64-column chunk (128 rows x 128 B)
static constexpr int kSmemBytes = kQBytes + kStages * 2 * kKVBytes + 1024 + 256;
static constexpr uint32_t kColS = 0, kColO = 128, kColP = 256;
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr float kRescaleThreshold = 8.0f;  // log2 domain: lazy rescale when max grows > 2^8

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

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ FwdMaps maps, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kQBytes;  // stage s: K at sKV + s*2*kKVBytes, V right after
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + kStages * 2 * kKVBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // kStages
  uint64_t* kv_empty = bars + 3;      // kStages
  uint64_t* s_full = bars + 5;        // 1
  uint64_t* p_full = bars + 6;        // 1   (4 arrivals: one per softmax warp)
  uint64_t* o_full = bars + 7;        // 1
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
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
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
    tmem_alloc(tmem_slot, 512);
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
      tma_load_3d(sQ, &maps.q, q_full, 0, kvh * G, q0);
      tma_load_3d(sQ + kChunk, &maps.q, q_full, 64, kvh * G, q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1u, abort_word)) break;
        uint8_t* sK = sKV + st * 2 * kKVBytes;
        uint8_t* sV = sK + kKVBytes;
        const int k0 = tile_index(j) * BN;
        mbar_arrive_expect_tx(&kv_full[st], 2 * kKVBytes);
        tma_load_3d(sK, &maps.k, &kv_full[st], 0, kvh, k0);
        tma_load_3d(sK + kChunk, &maps.k, &kv_full[st], 64, kvh, k0);
        tma_load_3d(sV, &maps.v, &kv_full[st], 0, kvh, k0);
        tma_load_3d(sV + kChunk, &maps.v, &kv_full[st], 64, kvh, k0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(BM, HD, 0, 1);   // P (TMEM)   x V (MN-major)
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_s = [&](int j) {
        const uint32_t k_addr = smem_u32(sKV + (j % kStages) * 2 * kKVBytes);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunk + (k & 3) * 32;
          tc_mma_ss(tmem + kColS, make_smem_desc(q_addr + off, 16, 1024),
                    make_smem_desc(k_addr + off, 16, 1024), idesc_s, k ? 1u : 0u);
        }
        tc_commit(s_full);
      };
      bool alive = mbar_wait(q_full, 0, abort_word) && mbar_wait(&kv_full[0], 0, abort_word);
      if (alive) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && alive; ++j) {
        if (j + 1 < n_tiles) {
          if (!mbar_wait(&kv_full[(j + 1) % kStages], ((j + 1) / kStages) & 1, abort_word)) break;
        }
        if (!mbar_wait(p_full, j & 1, abort_word)) break;
        tc_fence_after();
        if (j + 1 < n_tiles) issue_s(j + 1);
        const uint32_t v_addr = smem_u32(sKV + (j % kStages) * 2 * kKVBytes + kKVBytes);
        const uint32_t p_col = tmem + kColP + (j & 1) * 64;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          // V is MN-major: 64-wide dv chunks are kChunk apart, 16 keys = 2048 B.
          tc_mma_ts(tmem + kColO, p_col + k * 8, make_smem_desc(v_addr + k * 2048, kChunk, 1024),
                    idesc_o, (j | k) ? 1u : 0u);
        }
        tc_commit(&kv_empty[j % kStages]);
        tc_commit(o_full);
      }
    }
  } else {
    // ------------------------------------------------------- softmax --------
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    float m_used = -INFINITY, l_sum = 0.f;
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_word)) { alive = false; break; }
      tc_fence_after();
      const int k0 = tile_index(j) * BN;
      // visibility class of this tile for my row
      const int la = max(a0, k0), ha = min(a1, k0 + BN);
      const int lb = max(b0, k0), hb = min(b1, k0 + BN);
      const bool none = (ha <= la) && (hb <= lb);
      const bool full = (la == k0 && ha == k0 + BN) || (lb == k0 && hb == k0 + BN);
      // pass 1: row max
      float rmax = -INFINITY;
      if (!__all_sync(0xffffffffu, none)) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + lane_base + kColS + c, r);
          tmem_ld_wait();
          if (!none) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kk = k0 + c + i;
              const bool vis = full || (kk >= la && kk < ha) || (kk >= lb && kk < hb);
              if (vis) rmax = fmaxf(rmax, __uint_as_float(r[i]));
            }
          }
        }
      }
      rmax *= p.scale_log2;   // scale > 0; -inf stays -inf
      const float m_cand = fmaxf(m_used, rmax);
      const bool need = (m_cand > m_used) && (m_used == -INFINITY || m_cand - m_used > kRescaleThreshold);
      const float alpha = need ? (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_cand)) : 1.f;
      if (need) {
        m_used = m_cand;
        l_sum *= alpha;
      }
      // pass 2: P = exp2(s - m_used) -> TMEM (bf16 pairs), row sum
      const uint32_t p_addr = tmem + lane_base + kColP + (j & 1) * 64;
      float rsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN; c += 64) {
        uint32_t packed[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + lane_base + kColS + c + h * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float e[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int kk = k0 + c + h * 32 + i + u;
              const bool vis = !none && (full || (kk >= la && kk < ha) || (kk >= lb && kk < hb));
              e[u] = vis ? fast_exp2(__uint_as_float(r[i + u]) * p.scale_log2 - m_used) : 0.f;
            }
            // sum what the MMA will see (bf16-rounded) so the normaliser matches the numerator
            const uint32_t pk = pack_bf16x2(e[0], e[1]);
            const __nv_bfloat162 pb = *reinterpret_cast<const __nv_bfloat162*>(&pk);
            rsum += __low2float(pb) + __high2float(pb);
            packed[h * 16 + i / 2] = pk;
          }
        }
        // O must not be rescaled, and P_j not overwritten... P buffer j&1 was last read by PV_{j-2},
        // which completed before o_full of tile j-1 was observed in the previous iteration.
        tmem_st_32x32(p_addr + c / 2, packed);
      }
      l_sum += rsum;
      if (j > 0) {
        if (!mbar_wait(o_full, (j - 1) & 1, abort_word)) { alive = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tmem + lane_base + kColO + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(tmem + lane_base + kColO + c, r);
          }
        }
      }
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
        uint32_t r[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem + lane_base + kColO + c, r);
          tmem_ld_wait();
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            if (n_tiles > 0 && l_sum > 0.f) {
              o.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
              o.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
              o.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
              o.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
            } else {
              o = make_uint4(0, 0, 0, 0);
            }
            reinterpret_cast<uint4*>(orow + c)[i] = o;
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
    tmem_dealloc(tmem, 512);
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

// [rows, heads, 128] bf16 with row stride `ld` elements; box = 64 x box_heads x box_rows.
int make_map_rows_heads(CUtensorMap* map, const void* base, long long rows, int heads, long long ld,
                        int box_heads, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)ld * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

}  // namespace attn
}  // namespace ab

extern "C" int ab_attn_fwd(const void* q, const void* k, const void* v, const int* intervals, void* out,
                           float* lse, int q_total, int tk, int hq, int hkv, int head_dim,
                           long long k_ld, long long v_ld, float scale, int* status, void* stream) {
  using namespace ab;
  using namespace ab::attn;
  if (head_dim != HD || hq % hkv) return -10;
  const int G = hq / hkv;
  if (G > 16 || (BM % G)) return -11;
  if (q_total <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
    return -12;
  if ((k_ld & 7) || (v_ld & 7)) return -12;
  FwdMaps maps;
  const int pm = BM / G;
  int rc;
  if ((rc = make_map_rows_heads(&maps.q, q, q_total, hq, (long long)hq * HD, G, pm))) return rc;
  if ((rc = make_map_rows_heads(&maps.k, k, tk, hkv, k_ld, 1, BN))) return rc;
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
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return -3;
    attr_set = true;
  }
  dim3 grid((q_total + pm - 1) / pm, hkv);
  attn_fwd_kernel<<<grid, kThreads, kSmemBytes, reinterpret_cast<cudaStream_t>(stream)>>>(maps, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
