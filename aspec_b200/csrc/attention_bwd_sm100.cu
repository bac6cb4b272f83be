// Interval-masked flash attention backward for sm_100a (tcgen05 + TMEM + TMA).
//
// Three kernels:
//   attn_bwd_prep   delta[h, i] = sum_d O[i,h,d] dO[i,h,d], and per query tile the
//                   key ranges it can see (used by the dK/dV kernel to skip tiles)
//   attn_bwd_dq     one CTA per query tile (rows = positions x heads-in-group):
//                   S = Q K^T, dP = dO V^T, dS = P o (dP - delta) * scale, dQ += dS K
//   attn_bwd_dkv    one CTA per key tile of one key/value head; it walks the
//                   query tiles that see it:  S^T = K Q^T, dP^T = V dO^T,
//                   dV += P^T dO, dK += dS^T Q.  Because the G query heads of the
//                   group are folded into the row dimension, their contributions
//                   are summed on chip and dK / dV are written once, in bf16.
//
// P / dS are handed to the second MMA through tensor memory (bf16 pairs); in
// the dK/dV kernel they alias the S^T / dP^T columns they were computed from.
// Shared-memory tiles are used under two descriptor views: [rows, 64] K-major
// when the tile is the left/right operand of a d-reduction, and MN-major when
// the same bytes are the right operand of a row-reduction.
//
// Both main kernels are templates on the query/key head dimension HDQK: 128, or 192 for materialised-MLA heads
// (values stay 128 wide).  At 192 a dQ / dK accumulator would need 192 of the 512 tensor-memory columns next to S,
// dP and the other accumulators, so the grid gets a third dimension: pass 0 produces columns [0, 128) (and dV),
// pass 1 columns [128, 192); each pass recomputes S and dP.  The wider Q / K tiles also leave room for only one
// K/V (or Q/dO) stage in shared memory.
#include "common.cuh"

namespace ab {
namespace attn {

int make_map_rows_heads(CUtensorMap* map, const void* base, long long rows, int heads, long long ld,
                        int box_heads, int box_rows);
int make_map_rows_heads_d(CUtensorMap* map, const void* base, long long rows, int heads, long long ld,
                          int box_heads, int box_rows, int hd);

static constexpr int BM = 128;
static constexpr int BN = 128;
static constexpr int HD = 128;
static constexpr int kThreads = 320;   // TMA warp, MMA warp, two warpgroups that split every score tile by columns
static constexpr int kTile = 128 * HD * 2;   // 32 KB: one 128 x 128 bf16 tile (two swizzled chunks)
static constexpr int kChunk = 128 * 128;     // bytes per 64-column chunk
static constexpr float kLog2e = 1.4426950408889634f;

template <int HDQK> struct BwdCfg {
  static constexpr int kQKTile = 128 * HDQK * 2;                 // a Q or K tile: HDQK / 64 chunks
  static constexpr int kStages = HDQK == 128 ? 2 : 1;
  static constexpr int kPasses = (HDQK + 127) / 128;             // passes over the qk head dim for dQ / dK
  static constexpr int kDqSmem = kQKTile + kTile + kStages * (kQKTile + kTile) + 1024 + 256;
  static constexpr int kDkvSmem = kQKTile + kTile + kStages * (kQKTile + kTile) + 2 * 128 * 24 + 4096 * 4 + 1024 + 256;
};

struct BwdParams {
  const int* intervals;       // [Qtot, 4]
  const float* lse;           // [Hq, Qtot] natural log
  const float* delta;         // [Hq, Qtot]
  const int* tile_ranges;     // [n_qtiles, 4]  (c_lo, c_hi, b_lo, b_hi) in key index units
  __nv_bfloat16* dq;          // [Qtot, Hq, HDQK]
  __nv_bfloat16* dk;          // [Tk, Hkv, HDQK]
  __nv_bfloat16* dv;          // [Tk, Hkv, HD]
  int q_total, hq, hkv, group, tk, n_qtiles;
  float scale, scale_log2;
  int* status;
};
struct alignas(64) BwdMaps {
  CUtensorMap q, k, v, dout;
};

// ------------------------------------------------------------------ prep ----
// grid = ceil(Qtot / 8) x ...: one warp per (position, head): delta.  Block 0.. also ranges.
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ out,
                                     const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                     const int* __restrict__ intervals, int* __restrict__ tile_ranges,
                                     int q_total, int hq, int pm, int n_qtiles) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nw = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = w; r < (long long)q_total * hq; r += nw) {
    const uint2 a = reinterpret_cast<const uint2*>(out + r * HD)[lane];
    const uint2 b = reinterpret_cast<const uint2*>(dout + r * HD)[lane];
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(b2[i]);
      s += x.x * y.x + x.y * y.y;
    }
    s = warp_sum(s);
    if (lane == 0) {
      const long long pos = r / hq;
      const int h = (int)(r - pos * hq);
      delta[(size_t)h * q_total + pos] = s;
    }
  }
  // tile ranges: warp w handles query tile w
  for (long long t = w; t < n_qtiles; t += nw) {
    int c_lo = 0x7fffffff, c_hi = 0, b_lo = 0x7fffffff, b_hi = 0;
    for (int i = lane; i < pm; i += 32) {
      const long long pos = t * pm + i;
      if (pos < q_total) {
        const int4 iv = reinterpret_cast<const int4*>(intervals)[pos];
        if (iv.y > iv.x) { c_lo = min(c_lo, iv.x); c_hi = max(c_hi, iv.y); }
        if (iv.w > iv.z) { b_lo = min(b_lo, iv.z); b_hi = max(b_hi, iv.w); }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      c_lo = min(c_lo, __shfl_xor_sync(0xffffffffu, c_lo, o));
      c_hi = max(c_hi, __shfl_xor_sync(0xffffffffu, c_hi, o));
      b_lo = min(b_lo, __shfl_xor_sync(0xffffffffu, b_lo, o));
      b_hi = max(b_hi, __shfl_xor_sync(0xffffffffu, b_hi, o));
    }
    if (lane == 0) reinterpret_cast<int4*>(tile_ranges)[t] = make_int4(c_lo, c_hi, b_lo, b_hi);
  }
}

__device__ __forceinline__ bool visible(int kk, int a0, int a1, int b0, int b1) {
  return (kk >= a0 && kk < a1) || (kk >= b0 && kk < b1);
}

// -------------------------------------------------------------------- dQ ----
// TMEM: S [0,128)  dP [128,256)  dQ [256,384)  dS0 [384,448)  dS1 [448,512)
template <int HDQK>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ BwdMaps maps, const BwdParams p) {
  constexpr int kQKTile = BwdCfg<HDQK>::kQKTile, kStages = BwdCfg<HDQK>::kStages;
  constexpr int kStage = kQKTile + kTile;          // one K/V stage: K (HDQK wide) then V
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + kQKTile;
  uint8_t* sKV = sdO + kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + kStages * kStage);
  // this CTA's columns of dQ: [dcol0, dcol0 + ncols) of the HDQK-wide head
  const int dcol0 = blockIdx.z * 128;
  const int ncols = HDQK - dcol0 < 128 ? HDQK - dcol0 : 128;
  uint64_t* q_full = bars;        // Q and dO
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* sp_full = bars + 5;   // S and dP ready
  uint64_t* ds_full = bars + 6;   // dS written (4 arrivals)
  uint64_t* dq_done = bars + 7;   // [2] dQ MMA of tile j retired -> dq_done[j & 1] (frees dS buffer j & 1)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* range = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group, pm = BM / G;
  const int qt = gridDim.x - 1 - blockIdx.x;   // late tiles (longest prefixes) first
  const int q0 = qt * pm;
  const int kvh = blockIdx.y;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(sp_full, 1);
    mbar_init(ds_full, 8);
    mbar_init(&dq_done[0], 1);
    mbar_init(&dq_done[1], 1);
    fence_barrier_init();
    const int4 r = reinterpret_cast<const int4*>(p.tile_ranges)[qt];
    range[0] = r.x / BN; range[1] = (r.y + BN - 1) / BN;
    range[2] = r.z / BN; range[3] = (r.w + BN - 1) / BN;
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  int ca = range[0], cb = range[1], da = range[2], db = range[3];
  if (cb <= ca) { ca = 0; cb = 0; }
  if (db <= da) { da = 0; db = 0; }
  if (cb > ca && db > da) {
    if (da < ca) { int t0 = ca, t1 = cb; ca = da; cb = db; da = t0; db = t1; }
    if (da < cb) da = cb;
    if (db < da) db = da;
  }
  const int n_tiles = (cb - ca) + (db - da);
  auto tile_index = [&](int j) { return j < (cb - ca) ? ca + j : da + (j - (cb - ca)); };

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_arrive_expect_tx(q_full, kQKTile + kTile);
#pragma unroll
      for (int c = 0; c < HDQK / 64; ++c) tma_load_3d(sQ + c * kChunk, &maps.q, q_full, 64 * c, kvh * G, q0);
      tma_load_3d(sdO, &maps.dout, q_full, 0, kvh * G, q0);
      tma_load_3d(sdO + kChunk, &maps.dout, q_full, 64, kvh * G, q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kStages;
        if (!mbar_wait(&kv_empty[st], ((j / kStages) & 1) ^ 1u, abort_word)) break;
        uint8_t* sK = sKV + st * kStage;
        uint8_t* sV = sK + kQKTile;
        const int k0 = tile_index(j) * BN;
        mbar_arrive_expect_tx(&kv_full[st], kStage);
#pragma unroll
        for (int c = 0; c < HDQK / 64; ++c) tma_load_3d(sK + c * kChunk, &maps.k, &kv_full[st], 64 * c, kvh, k0);
        tma_load_3d(sV, &maps.v, &kv_full[st], 0, kvh, k0);
        tma_load_3d(sV + kChunk, &maps.v, &kv_full[st], 64, kvh, k0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(BM, BN, 0, 0);   // both K-major (d-reduction)
      const uint32_t idesc_dq = make_idesc_bf16(BM, ncols, 0, 1);    // dS (TMEM) x K (MN-major view), this pass's columns
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      auto issue_s_dp = [&](int j) {
        const uint32_t k_addr = smem_u32(sKV + (j % kStages) * kStage);
        const uint32_t v_addr = k_addr + kQKTile;
#pragma unroll
        for (int k = 0; k < HDQK / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunk + (k & 3) * 32;
          tc_mma_ss(tmem + 0, make_smem_desc(q_addr + off, 16, 1024),
                    make_smem_desc(k_addr + off, 16, 1024), idesc_kk, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunk + (k & 3) * 32;
          tc_mma_ss(tmem + 128, make_smem_desc(do_addr + off, 16, 1024),
                    make_smem_desc(v_addr + off, 16, 1024), idesc_kk, k ? 1u : 0u);
        }
        tc_commit(sp_full);
      };
      bool alive = mbar_wait(q_full, 0, abort_word);
      if (kStages == 2) {
        // S / dP of tile j + 1 are issued before dQ of tile j: the other K/V stage is already in shared memory
        alive = alive && mbar_wait(&kv_full[0], 0, abort_word);
        if (alive) { tc_fence_after(); issue_s_dp(0); }
        for (int j = 0; j < n_tiles && alive; ++j) {
          if (j + 1 < n_tiles && !mbar_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_word)) break;
          if (!mbar_wait(ds_full, j & 1, abort_word)) break;
          tc_fence_after();
          if (j + 1 < n_tiles) issue_s_dp(j + 1);
          const uint32_t k_addr = smem_u32(sKV + (j & 1) * kStage);
          const uint32_t ds_col = tmem + 384 + (j & 1) * 64;
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            tc_mma_ts(tmem + 256, ds_col + k * 8, make_smem_desc(k_addr + k * 2048, kChunk, 1024), idesc_dq,
                      (j | k) ? 1u : 0u);
          tc_commit(&kv_empty[j & 1]);
          tc_commit(&dq_done[j & 1]);
        }
      } else {
        // one K/V stage: the K tile is also the dQ MMA's operand, so a tile is finished before the next is loaded
        for (int j = 0; j < n_tiles && alive; ++j) {
          if (!mbar_wait(&kv_full[0], j & 1, abort_word)) break;
          tc_fence_after();
          issue_s_dp(j);
          if (!mbar_wait(ds_full, j & 1, abort_word)) break;
          tc_fence_after();
          const uint32_t k_addr = smem_u32(sKV) + (dcol0 / 64) * kChunk;   // this pass's 64-column chunks of K
          const uint32_t ds_col = tmem + 384 + (j & 1) * 64;
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            tc_mma_ts(tmem + 256, ds_col + k * 8, make_smem_desc(k_addr + k * 2048, kChunk, 1024), idesc_dq,
                      (j | k) ? 1u : 0u);
          tc_commit(&kv_empty[0]);
          tc_commit(&dq_done[j & 1]);
        }
      }
    }
  } else {
    // warps 2..9: TMEM lane quadrant warp % 4 (two warps per quadrant); the first four take score columns
    // [0, 64), the other four [64, 128) - no row reduction is needed in the backward pass
    const int qd = warp & 3;
    const int cbeg = ((warp - 2) >> 2) * 64;
    const uint32_t lane_base = static_cast<uint32_t>(qd * 32) << 16;
    const int t = qd * 32 + lane;
    const int pos = q0 + t / G;
    const int head = kvh * G + t % G;
    const bool row_ok = pos < p.q_total;
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
    float lse2 = 0.f, delta = 0.f;
    if (row_ok) {
      const int4 iv = reinterpret_cast<const int4*>(p.intervals)[pos];
      a0 = iv.x; a1 = iv.y; b0 = iv.z; b1 = iv.w;
      lse2 = p.lse[(size_t)head * p.q_total + pos] * kLog2e;
      delta = p.delta[(size_t)head * p.q_total + pos];
      if (!(lse2 > -INFINITY)) lse2 = 0.f;      // a row without any visible key: every score is masked to -inf below
    }
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      if (!mbar_wait(sp_full, j & 1, abort_word)) { alive = false; break; }
      // dS buffer j&1 was last read by the dQ MMA of tile j-2
      if (j >= 2 && !mbar_wait(&dq_done[j & 1], ((j >> 1) - 1) & 1, abort_word)) { alive = false; break; }
      tc_fence_after();
      const int k0 = tile_index(j) * BN;
      const uint32_t ds_addr = tmem + lane_base + 384 + (j & 1) * 64;
      // visible columns of this tile for my row, tile-local: [la, ha) U [lb, hb); a tile that every row of the warp
      // sees completely needs no per-element test
      const int la = max(a0 - k0, 0), ha = min(a1 - k0, BN);
      const int lb = max(b0 - k0, 0), hb = min(b1 - k0, BN);
      const uint32_t wa = (row_ok && ha > la) ? static_cast<uint32_t>(ha - la) : 0u;
      const uint32_t wb = (row_ok && hb > lb) ? static_cast<uint32_t>(hb - lb) : 0u;
      const bool warp_full = __all_sync(0xffffffffu, wa == BN || wb == BN);
      const float neg_lse = -lse2, neg_ds = -delta * p.scale;
#pragma unroll 1
      for (int c = cbeg; c < cbeg + 64; c += 32) {
        uint32_t s[32], dp[32], pk[16];
        tmem_ld_32x32(tmem + lane_base + c, s);
        tmem_ld_32x32(tmem + lane_base + 128 + c, dp);
        tmem_ld_wait();
        if (!warp_full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t col = static_cast<uint32_t>(c + i);
            const bool vis = (col - static_cast<uint32_t>(la) < wa) | (col - static_cast<uint32_t>(lb) < wb);
            s[i] = vis ? s[i] : 0xff800000u;        // exp2(-inf) = 0 -> dS = 0
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float pr = fast_exp2(fmaf(__uint_as_float(s[i + u]), p.scale_log2, neg_lse));
            e[u] = pr * fmaf(__uint_as_float(dp[i + u]), p.scale, neg_ds);
          }
          pk[i / 2] = pack_bf16x2(e[0], e[1]);
        }
        // 16 packed columns
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
            ::"r"(ds_addr + c / 2), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]),
            "r"(pk[6]), "r"(pk[7]), "r"(pk[8]), "r"(pk[9]), "r"(pk[10]), "r"(pk[11]), "r"(pk[12]),
            "r"(pk[13]), "r"(pk[14]), "r"(pk[15])
            : "memory");
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (alive && n_tiles > 0)
      alive = mbar_wait(&dq_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_word);
    if (alive) {
      tc_fence_after();
      __nv_bfloat16* row = p.dq + ((size_t)(row_ok ? pos : 0) * p.hq + head) * HDQK + dcol0;
#pragma unroll 1
      for (int c = cbeg; c < cbeg + 64 && c < ncols; c += 32) {
        uint32_t r[32];
        if (n_tiles > 0) { tmem_ld_32x32(tmem + lane_base + 256 + c, r); tmem_ld_wait(); }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o = make_uint4(0, 0, 0, 0);
            if (n_tiles > 0) {
              o.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
            }
            reinterpret_cast<uint4*>(row + c)[i] = o;
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
  if (warp == 1) { __syncwarp(); tmem_dealloc(tmem, 512); }
}

// ------------------------------------------------------------------ dK/dV ---
// TMEM: S^T / P^T [0,128)   dP^T / dS^T [128,256)   dV [256,384)   dK [384,512)
static constexpr int kListCap = 4096;

template <int HDQK>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ BwdMaps maps, const BwdParams p) {
  constexpr int kQKTile = BwdCfg<HDQK>::kQKTile, kStages = BwdCfg<HDQK>::kStages;
  constexpr int kStage = kQKTile + kTile;     // one Q/dO stage: Q (HDQK wide) then dO
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kQKTile;
  uint8_t* sQdO = sV + kTile;                 // stage s: Q at +s*kStage, dO right after
  uint8_t* meta = sQdO + kStages * kStage;    // buffer b: int4 iv[128]; float lse2[128]; float delta[128]
  // this CTA's columns of dK: [dcol0, dcol0 + ncols); dV belongs to pass 0
  const int dcol0 = blockIdx.z * 128;
  const int ncols = HDQK - dcol0 < 128 ? HDQK - dcol0 : 128;
  const bool with_dv = blockIdx.z == 0;
  int* list = reinterpret_cast<int*>(meta + 2 * 128 * 24);
  uint64_t* bars = reinterpret_cast<uint64_t*>(list + kListCap);
  uint64_t* kv_full = bars;         // 1
  uint64_t* qdo_full = bars + 1;    // [2]
  uint64_t* qdo_empty = bars + 3;   // [2]
  uint64_t* st_full = bars + 5;     // S^T and dP^T ready
  uint64_t* pds_full = bars + 6;    // P^T and dS^T written (4 arrivals)
  uint64_t* acc_done = bars + 7;    // dV/dK MMAs of the tile retired
  uint64_t* meta_bar = bars + 8;    // row metadata of the tile staged by all 128 softmax threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* n_list = reinterpret_cast<int*>(tmem_slot + 2);
  int* tile_cnt = reinterpret_cast<int*>(tmem_slot + 3);   // [2] running count of query rows that see the whole key tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group, pm = BM / G;
  const int k0 = blockIdx.x * BN;
  const int kvh = blockIdx.y;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    tile_cnt[0] = tile_cnt[1] = 0;
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
    mbar_init(st_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(acc_done, 1);
    mbar_init(meta_bar, 128);
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  if (warp == 0) {
    // Query tiles whose visible key ranges intersect [k0, k0 + BN): ordered compaction by ballot.
    int count = 0;
    for (int base = 0; base < p.n_qtiles; base += 32) {
      const int t = base + lane;
      bool hit = false;
      if (t < p.n_qtiles) {
        const int4 r = reinterpret_cast<const int4*>(p.tile_ranges)[t];
        hit = (r.y > r.x && r.x < k0 + BN && r.y > k0) || (r.w > r.z && r.z < k0 + BN && r.w > k0);
      }
      const uint32_t m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int idx = count + __popc(m & ((1u << lane) - 1));
        if (idx < kListCap) list[idx] = t;
      }
      count += __popc(m);
    }
    if (lane == 0) *n_list = count;   // the host guarantees n_qtiles <= kListCap
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n = *n_list;

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      mbar_arrive_expect_tx(kv_full, kQKTile + kTile);
#pragma unroll
      for (int c = 0; c < HDQK / 64; ++c) tma_load_3d(sK + c * kChunk, &maps.k, kv_full, 64 * c, kvh, k0);
      tma_load_3d(sV, &maps.v, kv_full, 0, kvh, k0);
      tma_load_3d(sV + kChunk, &maps.v, kv_full, 64, kvh, k0);
      for (int i = 0; i < n; ++i) {
        const int st = i % kStages;
        if (!mbar_wait(&qdo_empty[st], ((i / kStages) & 1) ^ 1u, abort_word)) break;
        uint8_t* sQ = sQdO + st * kStage;
        uint8_t* sdO = sQ + kQKTile;
        const int q0 = list[i] * pm;
        mbar_arrive_expect_tx(&qdo_full[st], kStage);
#pragma unroll
        for (int c = 0; c < HDQK / 64; ++c) tma_load_3d(sQ + c * kChunk, &maps.q, &qdo_full[st], 64 * c, kvh * G, q0);
        tma_load_3d(sdO, &maps.dout, &qdo_full[st], 0, kvh * G, q0);
        tma_load_3d(sdO + kChunk, &maps.dout, &qdo_full[st], 64, kvh * G, q0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(BN, BM, 0, 0);   // K/V (K-major) x Q/dO (K-major)
      constexpr uint32_t idesc_dv = make_idesc_bf16(BN, HD, 0, 1);   // P^T (TMEM) x dO (MN-major)
      const uint32_t idesc_dk = make_idesc_bf16(BN, ncols, 0, 1);    // dS^T (TMEM) x Q (MN-major), this pass's columns
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool alive = mbar_wait(kv_full, 0, abort_word);
      for (int i = 0; i < n && alive; ++i) {
        const int st = i % kStages;
        if (!mbar_wait(&qdo_full[st], (i / kStages) & 1, abort_word)) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQdO + st * kStage);
        const uint32_t do_addr = q_addr + kQKTile;
#pragma unroll
        for (int k = 0; k < HDQK / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunk + (k & 3) * 32;
          tc_mma_ss(tmem + 0, make_smem_desc(k_addr + off, 16, 1024),
                    make_smem_desc(q_addr + off, 16, 1024), idesc_kk, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunk + (k & 3) * 32;
          tc_mma_ss(tmem + 128, make_smem_desc(v_addr + off, 16, 1024),
                    make_smem_desc(do_addr + off, 16, 1024), idesc_kk, k ? 1u : 0u);
        }
        tc_commit(st_full);
        if (!mbar_wait(pds_full, i & 1, abort_word)) break;
        tc_fence_after();
#pragma unroll
        // Each warpgroup wrote its 64 query columns as 32 packed columns over scores IT had consumed:
        // query columns [0, 64) live at packed columns [0, 32), query columns [64, 128) at [64, 96).
        for (int k = 0; k < BM / 16; ++k)   // reduction over the 128 query rows of the tile
          if (with_dv)
            tc_mma_ts(tmem + 256, tmem + 0 + (k >> 2) * 64 + (k & 3) * 8, make_smem_desc(do_addr + k * 2048, kChunk, 1024),
                      idesc_dv, (i | k) ? 1u : 0u);
        const uint32_t qd_addr = q_addr + (dcol0 / 64) * kChunk;   // this pass's 64-column chunks of Q
#pragma unroll
        for (int k = 0; k < BM / 16; ++k)
          tc_mma_ts(tmem + 384, tmem + 128 + (k >> 2) * 64 + (k & 3) * 8, make_smem_desc(qd_addr + k * 2048, kChunk, 1024),
                    idesc_dk, (i | k) ? 1u : 0u);
        tc_commit(&qdo_empty[st]);
        tc_commit(acc_done);
      }
    }
  } else {
    // warps 2..9: TMEM lane quadrant warp % 4; the first four take query columns [0, 64) of every tile and stage
    // the tile's row metadata, the other four take columns [64, 128)
    const int qd = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int cbeg = wg * 64;
    const uint32_t lane_base = static_cast<uint32_t>(qd * 32) << 16;
    const int t = qd * 32 + lane;          // key row of the tile == TMEM lane
    const int kk = k0 + t;
    bool alive = true;
    int prev_cnt[2] = {0, 0};
    for (int i = 0; i < n && alive; ++i) {
      // Row metadata of query tile i (thread t fetches query row t) into shared memory.
      uint8_t* mb = meta + (i & 1) * 128 * 24;
      int4* m_iv = reinterpret_cast<int4*>(mb);
      float* m_lse = reinterpret_cast<float*>(mb + 128 * 16);
      float* m_delta = m_lse + 128;
      if (wg == 0) {
        const int pos = list[i] * pm + t / G;
        const int head = kvh * G + t % G;
        // per query row: interval starts and widths for the unsigned-compare visibility test, -lse (log2) and
        // -delta * scale; a query tile whose every row sees this whole key tile needs no per-element test
        uint4 iv = make_uint4(0u, 0u, 0u, 0u);
        float l2 = 0.f, dl = 0.f;
        bool covers = false;
        if (pos < p.q_total) {
          const int4 raw = reinterpret_cast<const int4*>(p.intervals)[pos];
          iv = make_uint4((uint32_t)raw.x, raw.y > raw.x ? (uint32_t)(raw.y - raw.x) : 0u, (uint32_t)raw.z,
                          raw.w > raw.z ? (uint32_t)(raw.w - raw.z) : 0u);
          l2 = p.lse[(size_t)head * p.q_total + pos] * kLog2e;
          if (!(l2 > -INFINITY)) l2 = 0.f;
          dl = p.delta[(size_t)head * p.q_total + pos];
          covers = (raw.x <= k0 && raw.y >= k0 + BN) || (raw.z <= k0 && raw.w >= k0 + BN);
        }
        reinterpret_cast<uint4*>(m_iv)[t] = iv;
        m_lse[t] = -l2;
        m_delta[t] = -dl * p.scale;
        if (covers) atomicAdd(&tile_cnt[i & 1], 1);
        mbar_arrive(meta_bar);
      }
      if (!mbar_wait(meta_bar, i & 1, abort_word)) { alive = false; break; }
      // the counter only grows; it is next touched at tile i + 2, after every thread has passed the barrier of
      // tile i + 1, hence after this read
      const int seen = *reinterpret_cast<volatile int*>(&tile_cnt[i & 1]);
      const bool all_full = (seen - prev_cnt[i & 1]) == 128;
      prev_cnt[i & 1] = seen;
      if (!mbar_wait(st_full, i & 1, abort_word)) { alive = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = cbeg; c < cbeg + 64; c += 32) {
        uint32_t s[32], dp[32], pp[16], ds[16];
        tmem_ld_32x32(tmem + lane_base + c, s);
        tmem_ld_32x32(tmem + lane_base + 128 + c, dp);
        tmem_ld_wait();
        if (!all_full) {
#pragma unroll
          for (int r = 0; r < 32; ++r) {
            const uint4 iv = reinterpret_cast<const uint4*>(m_iv)[c + r];
            const bool vis = ((uint32_t)kk - iv.x < iv.y) | ((uint32_t)kk - iv.z < iv.w);
            s[r] = vis ? s[r] : 0xff800000u;
          }
        }
#pragma unroll
        for (int r = 0; r < 32; r += 4) {
          const float4 nl = *reinterpret_cast<const float4*>(m_lse + c + r);
          const float4 nd = *reinterpret_cast<const float4*>(m_delta + c + r);
          const float nls[4] = {nl.x, nl.y, nl.z, nl.w}, nds[4] = {nd.x, nd.y, nd.z, nd.w};
          float pv[4], dsv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            pv[u] = fast_exp2(fmaf(__uint_as_float(s[r + u]), p.scale_log2, nls[u]));
            dsv[u] = pv[u] * fmaf(__uint_as_float(dp[r + u]), p.scale, nds[u]);
          }
          pp[r / 2] = pack_bf16x2(pv[0], pv[1]);
          pp[r / 2 + 1] = pack_bf16x2(pv[2], pv[3]);
          ds[r / 2] = pack_bf16x2(dsv[0], dsv[1]);
          ds[r / 2 + 1] = pack_bf16x2(dsv[2], dsv[3]);
        }
        // P^T over the S^T columns already consumed, dS^T over the dP^T columns already consumed
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
            ::"r"(tmem + lane_base + cbeg + (c - cbeg) / 2), "r"(pp[0]), "r"(pp[1]), "r"(pp[2]), "r"(pp[3]), "r"(pp[4]),
            "r"(pp[5]), "r"(pp[6]), "r"(pp[7]), "r"(pp[8]), "r"(pp[9]), "r"(pp[10]), "r"(pp[11]),
            "r"(pp[12]), "r"(pp[13]), "r"(pp[14]), "r"(pp[15])
            : "memory");
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
            ::"r"(tmem + lane_base + 128 + cbeg + (c - cbeg) / 2), "r"(ds[0]), "r"(ds[1]), "r"(ds[2]), "r"(ds[3]),
            "r"(ds[4]), "r"(ds[5]), "r"(ds[6]), "r"(ds[7]), "r"(ds[8]), "r"(ds[9]), "r"(ds[10]),
            "r"(ds[11]), "r"(ds[12]), "r"(ds[13]), "r"(ds[14]), "r"(ds[15])
            : "memory");
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    if (alive && n > 0) alive = mbar_wait(acc_done, (n - 1) & 1, abort_word);
    if (alive) {
      tc_fence_after();
      const bool row_ok = kk < p.tk;
      __nv_bfloat16* dvrow = p.dv + ((size_t)(row_ok ? kk : 0) * p.hkv + kvh) * HD;
      __nv_bfloat16* dkrow = p.dk + ((size_t)(row_ok ? kk : 0) * p.hkv + kvh) * HDQK + dcol0;
#pragma unroll 1
      for (int half = with_dv ? 0 : 1; half < 2; ++half) {
        __nv_bfloat16* row = half ? dkrow : dvrow;
        const uint32_t col0 = half ? 384 : 256;
        const int width = half ? ncols : HD;
#pragma unroll 1
        for (int c = cbeg; c < cbeg + 64 && c < width; c += 32) {
          uint32_t r[32];
          if (n > 0) { tmem_ld_32x32(tmem + lane_base + col0 + c, r); tmem_ld_wait(); }
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o = make_uint4(0, 0, 0, 0);
              if (n > 0) {
                o.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                o.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                o.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                o.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
              }
              reinterpret_cast<uint4*>(row + c)[i] = o;
            }
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
  if (warp == 1) { __syncwarp(); tmem_dealloc(tmem, 512); }
}

}  // namespace attn
}  // namespace ab

template <int HDQK>
static int launch_bwd_main(const ab::attn::BwdMaps& maps, const ab::attn::BwdParams& p, int n_qtiles, int n_ktiles,
                           cudaStream_t stream) {
  using namespace ab;
  using namespace ab::attn;
  using Cfg = BwdCfg<HDQK>;
  static std::atomic<unsigned long long> attr_done{0};
  if (!once_per_device(attr_done, [&] {
        return cudaFuncSetAttribute(attn_bwd_dq_kernel<HDQK>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kDqSmem) == cudaSuccess &&
               cudaFuncSetAttribute(attn_bwd_dkv_kernel<HDQK>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kDkvSmem) == cudaSuccess;
      }))
    return -3;
  attn_bwd_dq_kernel<HDQK><<<dim3(n_qtiles, p.hkv, Cfg::kPasses), kThreads, Cfg::kDqSmem, stream>>>(maps, p);
  attn_bwd_dkv_kernel<HDQK><<<dim3(n_ktiles, p.hkv, Cfg::kPasses), kThreads, Cfg::kDkvSmem, stream>>>(maps, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// `head_dim` is the query/key head dimension (128, or 192 for materialised-MLA heads); values, out and dout are 128
// wide.  dq [Qtot,Hq,head_dim], dk [Tk,Hkv,head_dim], dv [Tk,Hkv,128] contiguous bf16.  Scratch supplied by the caller
// and filled here: delta [Hq,Qtot] fp32 and ranges [ceil(Qtot / (128 / G)), 4] int32.
extern "C" int ab_attn_bwd(const void* q, const void* k, const void* v, const int* intervals,
                           const void* out, const float* lse, const void* dout, float* delta,
                           int* ranges, void* dq,
                           void* dk, void* dv, int q_total, int tk, int hq, int hkv, int head_dim,
                           long long k_ld, long long v_ld, float scale, int* status, void* stream_) {
  using namespace ab;
  using namespace ab::attn;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if ((head_dim != HD && head_dim != 192) || hq % hkv) return -10;
  const int G = hq / hkv;
  if (G > 16 || (BM % G)) return -11;
  if (q_total <= 0 || tk <= 0) return 0;
  const int pm = BM / G;
  const int n_qtiles = (q_total + pm - 1) / pm;
  const int n_ktiles = (tk + BN - 1) / BN;
  if (n_qtiles > kListCap) return -15;
  long long prep_blocks = ((long long)q_total * hq + 7) / 8;
  if (prep_blocks > 148 * 8) prep_blocks = 148 * 8;
  attn_bwd_prep_kernel<<<(int)prep_blocks, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta,
      intervals, ranges, q_total, hq, pm, n_qtiles);
  BwdMaps maps;
  int rc;
  if ((rc = make_map_rows_heads_d(&maps.q, q, q_total, hq, (long long)hq * head_dim, G, pm, head_dim))) return rc;
  if ((rc = make_map_rows_heads(&maps.dout, dout, q_total, hq, (long long)hq * HD, G, pm))) return rc;
  if ((rc = make_map_rows_heads_d(&maps.k, k, tk, hkv, k_ld, 1, BN, head_dim))) return rc;
  if ((rc = make_map_rows_heads(&maps.v, v, tk, hkv, v_ld, 1, BN))) return rc;
  BwdParams p;
  p.intervals = intervals;
  p.lse = lse;
  p.delta = delta;
  p.tile_ranges = ranges;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.q_total = q_total;
  p.hq = hq;
  p.hkv = hkv;
  p.group = G;
  p.tk = tk;
  p.n_qtiles = n_qtiles;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.status = status;
  return head_dim == HD ? launch_bwd_main<128>(maps, p, n_qtiles, n_ktiles, stream)
                        : launch_bwd_main<192>(maps, p, n_qtiles, n_ktiles, stream);
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that cannot allocate (see aspec_b200_noalloc.h for who they are and why).
// The scratch that ab_attn_bwd takes from its caller lives here instead, in module memory.
#include "aspec_b200_noalloc.h"

#include <mutex>

namespace {

// delta [hq * q_total] fp32 first, then the per-query-tile key ranges [tiles, 4] int32.
static __device__ __align__(256) unsigned char g_noalloc_scratch[AB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
unsigned char* g_noalloc_ptr[kMaxDevices] = {nullptr};   // device address of the block, per GPU
std::mutex g_noalloc_mutex;

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device
// current.
unsigned char* noalloc_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) return nullptr;
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(ptr);
  }
  return g_noalloc_ptr[dev];
}

}  // namespace

extern "C" int ab_attn_bwd_static_scratch(const void* q, const void* k, const void* v,
                                          const int* intervals, const void* out, const float* lse,
                                          const void* dout, void* dq, void* dk, void* dv, int q_total,
                                          int tk, int hq, int hkv, int head_dim, long long k_ld,
                                          long long v_ld, float scale, int* status, void* stream) {
  if (q_total <= 0 || tk <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || hq % hkv) return -10;
  const int group = hq / hkv;
  if (group > 16 || (128 % group)) return -11;
  const int positions_per_tile = 128 / group;
  const long long tiles = ((long long)q_total + positions_per_tile - 1) / positions_per_tile;
  if ((long long)hq * q_total > AB_NOALLOC_MAX_ROW_STATS || tiles > AB_NOALLOC_MAX_QUERY_TILES)
    return AB_NOALLOC_TOO_LARGE;   // larger than the built-in scratch block: nothing is launched
  unsigned char* base = noalloc_scratch_for_current_device();
  if (!base) return AB_NOALLOC_SETUP_FAILED;
  float* delta = reinterpret_cast<float*>(base);
  int* ranges = reinterpret_cast<int*>(base + (size_t)AB_NOALLOC_MAX_ROW_STATS * 4);
  // Every word of delta / ranges that the two main kernels read is written by the preparation
  // kernel of this same call, so stale contents from an earlier call are never observed.
  return ab_attn_bwd(q, k, v, intervals, out, lse, dout, delta, ranges, dq, dk, dv, q_total, tk, hq, hkv,
                     head_dim, k_ld, v_ld, scale, status, stream);
}
