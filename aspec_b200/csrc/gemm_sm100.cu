// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] = sum_s  A_s[M,K_s] * B_s[N,K_s]^T      (s = 0, or 0..1 "dual source")
//
// * operands are staged by TMA into 128-byte-swizzled shared memory tiles,
// * one elected thread issues tcgen05.mma (128 x 256 x 16, bf16 -> fp32),
// * the fp32 accumulator lives in tensor memory (two 256-column buffers so the
//   epilogue of tile i overlaps the main loop of tile i+1),
// * four epilogue warps read the accumulator back with tcgen05.ld.
//
// Either operand may be K-major (the reduction index is contiguous in global
// memory: x[M,K], W[N,K] of a Linear forward) or MN-major (the output index is
// contiguous: the same W[N,K] read as the B operand of dX = dY * W, or dY / X
// read as operands of dW = dY^T * X), so forward, input-gradient and
// weight-gradient GEMMs all run without a transposed copy.
//
// Epilogues (template parameter):
//   EPI_STORE      D -> bf16 (or fp32), optional "+= C" residual / accumulate
//   EPI_ROWSTATS   D -> bf16 logits, plus per (row, n-tile) softmax partials
//                  (max, sum exp) in fp32: the vocabulary-head forward
//   EPI_SWIGLU     B holds gate/up rows interleaved in blocks of 128 output
//                  columns per half; D -> silu(gate) * up in bf16
//
// All waits are bounded (common.cuh); a timeout is reported in status[0].
#include <cstdio>
#include <cstdlib>
#include "common.cuh"

#include <stdio.h>

namespace ab {

static constexpr int BM = 128;
static constexpr int BN = 256;
static constexpr int BK = 64;          // 64 bf16 = one 128-byte swizzle row
static constexpr int UMMA_K = 16;
static constexpr int kStages = 4;
static constexpr int kAccBufs = 2;
static constexpr int kTmemCols = 512;  // 2 x 256 fp32 columns
static constexpr int kThreads = 192;   // warp0 TMA, warp1 MMA, warps 2..5 epilogue
static constexpr int kATileBytes = BM * BK * 2;
static constexpr int kBTileBytes = BN * BK * 2;
static constexpr int kStageBytes = kATileBytes + kBTileBytes;
static constexpr int kStoreStageBytes = 4 * 32 * 256;  // per epilogue warp: 32 rows x 128 bf16 columns, for row-contiguous stores
static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/ + kStoreStageBytes;

enum { EPI_STORE = 0, EPI_ROWSTATS = 1, EPI_SWIGLU = 2 };

struct GemmParams {
  int M, N;
  int k_blocks0;        // K_0 / 64 (rounded up)
  int k_blocks1;        // K_1 / 64 (0 when single source)
  int m_tiles, n_tiles;
  // output
  void* D;              // bf16 or fp32, row-major, leading dimension ldd
  long long ldd;
  int d_is_fp32;
  const void* C;        // optional addend with the layout and type of D
  float alpha;          // D = alpha * acc (+ C)
  // EPI_ROWSTATS: partial softmax statistics [n_tiles, M, 2] fp32
  float* stats;
  float logit_scale;    // logits = acc * logit_scale (applied before stats/store)
  int* status;
  // Stream-K: every CTA takes an equal, contiguous share of the (tile, k-block) space.  A tile whose
  // k-range is split over CTAs is combined with fp32 atomic adds (D is fp32 and either zeroed by the
  // caller or equal to C, the in-place accumulate case).
  // Up to kMaxMirrors extra bf16 destinations that receive the same tile (EPI_STORE, bf16): the Target's
  // captured-layer epilogue writes the residual stream to its own buffer and straight into the ring
  // slots of the consuming Draft ranks (peer memory mapped into this process, plain st.global over
  // NVLink).  mirror_ld is the row stride in elements.
  void* mirror[8];
  long long mirror_ld[8];
  int n_mirrors;
  // mirror_cols > 0: scatter instead of broadcast - output columns [m * mirror_cols, (m + 1) * mirror_cols) go ONLY
  // to mirror[m], at column (col % mirror_cols); D itself is not written (sequence<->head all-to-all in the epilogue).
  int mirror_cols;
  int stream_k;
  int full_tiles;
  long long units_per_cta;
};

struct alignas(64) GemmMaps {
  CUtensorMap a0, b0, a1, b1;
};

// Tile order: n-tile major, m-tile minor.  A wave of CTAs shares a handful of
// B (weight) tiles while A (activations, small) stays in L2, so the weight
// matrix is streamed from HBM once.
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int& mt, int& nt) {
  nt = tile / m_tiles;
  mt = tile - nt * m_tiles;
}

// Work iterator shared by the three warp roles.
// Phase 1 (always): whole tiles, strided by the grid, for the `full_tiles` tiles that fill complete
// waves.  Concurrent CTAs then walk the reduction dimension in step, so the A / B k-slabs they share
// are fetched from HBM once and served from L2.
// Phase 2 (stream-K only): the tiles of the last, partial wave are cut along K into equal contiguous
// shares, one per CTA; those split tiles are combined with fp32 reductions.
struct Work {
  long long cur;
  int in_tail;
};
// `unit` / `units`: index and number of schedulers walking the tile space (CTAs, or CTA pairs).
__device__ __forceinline__ Work work_begin(int unit) {
  Work w;
  w.cur = unit;
  w.in_tail = 0;
  return w;
}
__device__ __forceinline__ bool next_work(const GemmParams& p, int total_tiles, int k_blocks, Work& w, int unit,
                                          int units, int& tile, int& kb0, int& kb1) {
  const int full_tiles = p.stream_k ? p.full_tiles : total_tiles;
  if (!w.in_tail) {
    if (w.cur < full_tiles) {
      tile = (int)w.cur;
      kb0 = 0;
      kb1 = k_blocks;
      w.cur += units;
      return true;
    }
    if (!p.stream_k) return false;
    w.in_tail = 1;
    w.cur = (long long)unit * p.units_per_cta;
  }
  long long end = ((long long)unit + 1) * p.units_per_cta;
  const long long total = (long long)(total_tiles - full_tiles) * k_blocks;
  if (end > total) end = total;
  if (w.cur >= end) return false;
  const int t = (int)(w.cur / k_blocks);
  tile = full_tiles + t;
  kb0 = (int)(w.cur - (long long)t * k_blocks);
  long long seg_end = ((long long)t + 1) * k_blocks;
  if (seg_end > end) seg_end = end;
  kb1 = kb0 + (int)(seg_end - w.cur);
  w.cur = seg_end;
  return true;
}

// PAIR = 1: two CTAs of a cluster share every 256 x 256 output tile (tcgen05 cta_group::2).  Each stages its own
// 128 rows of A and its own 128-column half of B (32 KB per k-block instead of 48 KB, six stages instead of four),
// the even CTA issues the 256-row MMAs, each CTA keeps and drains its own 128 accumulator rows.  Barriers: tile
// loads of both CTAs report their bytes to the even CTA's full barrier; the MMA thread commits to the empty and
// accumulator-full barriers of both CTAs; the epilogue warps of both CTAs arrive on the even CTA's accumulator-empty
// barrier.  No load requests cluster multicast.
template <int A_MN, int B_MN, int EPI, int PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p) {
  constexpr int NS = PAIR ? 6 : kStages;                       // pipeline stages
  constexpr int BN_LOAD = PAIR ? BN / 2 : BN;                  // B rows (output columns) staged by this CTA
  constexpr int STAGE = kATileBytes + BN_LOAD * BK * 2;        // bytes per stage in this CTA
  static_assert(NS * STAGE == kStages * kStageBytes, "both layouts fill the same shared-memory budget");
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int units = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atom (8 rows x 128 B).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;                  // [NS]
  uint64_t* empty_bar = bars + NS;            // [NS]
  uint64_t* acc_full = bars + 2 * NS;         // [kAccBufs]
  uint64_t* acc_empty = bars + 2 * NS + kAccBufs;  // [kAccBufs]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NS + 2 * kAccBufs);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.m_tiles * p.n_tiles;
  const int k_blocks = p.k_blocks0 + p.k_blocks1;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], PAIR ? 8 : 4);  // one arrive per epilogue warp (of both CTAs of a pair)
    }
    fence_barrier_init();
    tma_prefetch_desc(&maps.a0);
    tma_prefetch_desc(&maps.b0);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the other CTA's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer ---------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      Work cursor = work_begin(unit);
      int tile, kb0, kb1;
      while (alive && next_work(p, total_tiles, k_blocks, cursor, unit, units, tile, kb0, kb1)) {
        int mt, nt;
        tile_coords(tile, p.m_tiles, mt, nt);
        const int row0 = (PAIR ? mt * 2 + (int)cta_rank : mt) * BM;       // this CTA's rows of A
        const int col0 = nt * BN + (PAIR ? (int)cta_rank * BN_LOAD : 0);  // this CTA's rows of B
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word)) { alive = false; break; }
          const bool second = kb >= p.k_blocks0;
          const CUtensorMap* ma = second ? &maps.a1 : &maps.a0;
          const CUtensorMap* mb = second ? &maps.b1 : &maps.b0;
          const int k0 = (second ? kb - p.k_blocks0 : kb) * BK;
          uint8_t* sa = smem + stage * STAGE;
          uint8_t* sb = sa + kATileBytes;
          if (PAIR) {
            // both CTAs' bytes are counted on the even CTA's barrier, which alone expects them
            const uint32_t bar0 = mapa_u32(smem_u32(&full_bar[stage]), 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_2d_pair(sa + j * (BK * 128), ma, bar0, row0 + j * 64, k0);
            } else {
              tma_load_2d_pair(sa, ma, bar0, k0, row0);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN_LOAD / 64; ++j)
                tma_load_2d_pair(sb + j * (BK * 128), mb, bar0, col0 + j * 64, k0);
            } else {
              tma_load_2d_pair(sb, mb, bar0, k0, col0);
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], STAGE);
            if (A_MN) {
              // global A^T is [K, M] row-major: box = 64 (m) x 64 (k rows)
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_2d(sa + j * (BK * 128), ma, &full_bar[stage], row0 + j * 64, k0);
            } else {
              tma_load_2d(sa, ma, &full_bar[stage], k0, row0);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (BK * 128), mb, &full_bar[stage], col0 + j * 64, k0);
            } else {
              tma_load_2d(sb, mb, &full_bar[stage], k0, col0);
            }
          }
          if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer -----------
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(PAIR ? 2 * BM : BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      Work cursor = work_begin(unit);
      int tile, kb0, kb1;
      while (alive && next_work(p, total_tiles, k_blocks, cursor, unit, units, tile, kb0, kb1)) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_word)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE);
          const uint32_t sb = sa + kATileBytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: advance 16 elements = 32 B inside the swizzle row.
            // MN-major: advance 16 k-rows of 128 B = 2048 B.
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            if (PAIR)
              tc_mma_ss_pair(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            else
              tc_mma_ss(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          // frees the smem stage (in both CTAs of a pair) when the MMAs retire
          if (PAIR) {
            tc_commit_pair(smem_u32(&empty_bar[stage]));
            tc_commit_pair(mapa_u32(smem_u32(&empty_bar[stage]), 1));
          } else {
            tc_commit(&empty_bar[stage]);
          }
          if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
        if (alive) {
          if (PAIR) {
            tc_commit_pair(smem_u32(&acc_full[acc]));
            tc_commit_pair(mapa_u32(smem_u32(&acc_full[acc]), 1));
          } else {
            tc_commit(&acc_full[acc]);
          }
        }
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------ epilogue warps -------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    Work cursor = work_begin(unit);
    int tile, kb0, kb1;
    while (next_work(p, total_tiles, k_blocks, cursor, unit, units, tile, kb0, kb1)) {
      int mt, nt;
      tile_coords(tile, p.m_tiles, mt, nt);
      if (PAIR) mt = mt * 2 + (int)cta_rank;   // this CTA's 128 rows of the pair's 256
      const bool partial = p.stream_k && !(kb0 == 0 && kb1 == k_blocks);
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_word)) break;
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
      const int col0 = nt * BN;

      if (EPI == EPI_ROWSTATS) {
        // Online softmax partials over this tile's 256 columns + bf16 logits.
        float run_max = -INFINITY, run_sum = 0.f;
        const float sc = p.logit_scale;
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)row * p.ldd;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c, r);
          tmem_ld_wait();
          float v[32];
          float cmax = -INFINITY;
          const int ncol = p.N - (col0 + c);  // valid columns in this chunk
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // Statistics are taken on the bf16-rounded value that is stored, so
            // that the loss kernel sees exactly the distribution normalised here.
            float x = __bfloat162float(__float2bfloat16(__uint_as_float(r[i]) * sc));
            v[i] = (i < ncol) ? x : -INFINITY;
            cmax = fmaxf(cmax, v[i]);
          }
          const float new_max = fmaxf(run_max, cmax);
          if (new_max > -INFINITY) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) s += fast_exp2((v[i] - new_max) * 1.4426950408889634f);
            run_sum = run_sum * fast_exp2((run_max - new_max) * 1.4426950408889634f) + s;
            run_max = new_max;
          }
          if (row_ok && ncol > 0) {
            if (ncol >= 32 && (p.ldd & 7) == 0) {
              uint4* dst = reinterpret_cast<uint4*>(drow + col0 + c);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 o;
                o.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
                o.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
                o.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
                dst[i] = o;
              }
            } else {
              for (int i = 0; i < 32 && i < ncol; ++i) drow[col0 + c + i] = __float2bfloat16(v[i]);
            }
          }
        }
        if (row_ok) {
          float2* st = reinterpret_cast<float2*>(p.stats) + ((long long)nt * p.M + row);
          *st = make_float2(run_max, run_sum);
        }
      } else if (EPI == EPI_SWIGLU) {
        // Columns [0,128) of the tile are gate, [128,256) the matching up rows.
        __nv_bfloat16* drow =
            reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)row * p.ldd + nt * (BN / 2);
        const int n_half = p.N / 2;
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_row + c, g);
          tmem_ld_32x32(t_row + BN / 2 + c, u);
          tmem_ld_wait();
          const int ncol = n_half - (nt * (BN / 2) + c);
          if (row_ok && ncol > 0) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float gf = __uint_as_float(g[i]);
              const float uf = __uint_as_float(u[i]);
              v[i] = gf / (1.f + __expf(-gf)) * uf;
            }
            if (ncol >= 32 && (p.ldd & 7) == 0) {
              uint4* dst = reinterpret_cast<uint4*>(drow + c);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 o;
                o.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
                o.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
                o.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
                dst[i] = o;
              }
            } else {
              for (int i = 0; i < 32 && i < ncol; ++i) drow[c + i] = __float2bfloat16(v[i]);
            }
          }
        }
      } else {
        const float alpha = p.alpha;
        // Tiles that also go to other destinations (peer memory over NVLink) are transposed through shared memory so
        // that every store instruction writes two whole 256-byte row segments instead of 32 scattered 16-byte pieces:
        // a link carries full sectors only when a warp's stores are contiguous.
        const bool staged = p.n_mirrors > 0 && !p.d_is_fp32 && !partial && col0 + BN <= p.N;
        if (staged) {
          uint8_t* stg = smem + kStages * kStageBytes + 256 + q * (32 * 256);
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
              uint32_t r[32];
              const int c = half * 128 + cc * 32;
              tmem_ld_32x32(t_row + c, r);
              tmem_ld_wait();
              const __nv_bfloat16* crow =
                  (p.C && row_ok) ? reinterpret_cast<const __nv_bfloat16*>(p.C) + (long long)row * p.ldd + col0 + c : nullptr;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[8 * i + j]) * alpha;
                if (crow) {
                  const uint4 cv = reinterpret_cast<const uint4*>(crow)[i];
                  const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&cv);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(c2[j]);
                    v[2 * j] += f.x;
                    v[2 * j + 1] += f.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(v[0], v[1]);
                o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]);
                o.w = pack_bf16x2(v[6], v[7]);
                const int chunk = cc * 4 + i;  // 16-byte piece of this lane's 256-byte row segment, XOR-swizzled
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
              }
            }
            __syncwarp();
#pragma unroll 1
            for (int r2 = 0; r2 < 16; ++r2) {
              const int rr = 2 * r2 + (lane >> 4);
              const int ch = lane & 15;
              const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((ch ^ (rr & 15)) << 4));
              const int grow = mt * BM + q * 32 + rr;
              if (grow < p.M) {
                const int gcol = col0 + half * 128 + ch * 8;
                if (p.mirror_cols > 0) {
                  const int dst = gcol / p.mirror_cols;
                  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.mirror[dst]) +
                                            (long long)grow * p.mirror_ld[dst] + (gcol - dst * p.mirror_cols)) = o;
                } else {
                  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)grow * p.ldd + gcol) = o;
                  for (int m = 0; m < p.n_mirrors; ++m)
                    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.mirror[m]) +
                                              (long long)grow * p.mirror_ld[m] + gcol) = o;
                }
              }
            }
            __syncwarp();
          }
        }
#pragma unroll 1
        for (int c = staged ? BN : 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c, r);
          tmem_ld_wait();
          const int ncol = p.N - (col0 + c);
          if (row_ok && ncol > 0 && partial) {
            // part of a split tile: combine in fp32 with vector reductions
            float* drow = reinterpret_cast<float*>(p.D) + (long long)row * p.ldd + col0 + c;
            if (ncol >= 32 && (p.ldd & 3) == 0) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(drow + 4 * i),
                             "f"(__uint_as_float(r[4 * i]) * alpha), "f"(__uint_as_float(r[4 * i + 1]) * alpha),
                             "f"(__uint_as_float(r[4 * i + 2]) * alpha), "f"(__uint_as_float(r[4 * i + 3]) * alpha)
                             : "memory");
            } else {
              for (int i = 0; i < 32 && i < ncol; ++i) atomicAdd(drow + i, __uint_as_float(r[i]) * alpha);
            }
          } else if (row_ok && ncol > 0) {
            if (p.d_is_fp32) {
              float* drow = reinterpret_cast<float*>(p.D) + (long long)row * p.ldd + col0 + c;
              const float* crow =
                  p.C ? reinterpret_cast<const float*>(p.C) + (long long)row * p.ldd + col0 + c
                      : nullptr;
              if (ncol >= 32 && (p.ldd & 3) == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  float4 o = make_float4(__uint_as_float(r[4 * i]) * alpha,
                                         __uint_as_float(r[4 * i + 1]) * alpha,
                                         __uint_as_float(r[4 * i + 2]) * alpha,
                                         __uint_as_float(r[4 * i + 3]) * alpha);
                  if (crow) {
                    const float4 cc = reinterpret_cast<const float4*>(crow)[i];
                    o.x += cc.x; o.y += cc.y; o.z += cc.z; o.w += cc.w;
                  }
                  reinterpret_cast<float4*>(drow)[i] = o;
                }
              } else {
                for (int i = 0; i < 32 && i < ncol; ++i)
                  drow[i] = __uint_as_float(r[i]) * alpha + (crow ? crow[i] : 0.f);
              }
            } else {
              if (p.mirror_cols > 0) {
                // scatter: this 32-column chunk belongs to exactly one destination
                const int gcol = col0 + c;
                const int dst = gcol / p.mirror_cols;
                __nv_bfloat16* mrow = reinterpret_cast<__nv_bfloat16*>(p.mirror[dst]) +
                                      (long long)row * p.mirror_ld[dst] + (gcol - dst * p.mirror_cols);
                if (ncol >= 32) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    uint4 o;
                    o.x = pack_bf16x2(__uint_as_float(r[8 * i]) * alpha, __uint_as_float(r[8 * i + 1]) * alpha);
                    o.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * alpha, __uint_as_float(r[8 * i + 3]) * alpha);
                    o.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * alpha, __uint_as_float(r[8 * i + 5]) * alpha);
                    o.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * alpha, __uint_as_float(r[8 * i + 7]) * alpha);
                    reinterpret_cast<uint4*>(mrow)[i] = o;
                  }
                } else {
                  for (int i = 0; i < ncol; ++i) mrow[i] = __float2bfloat16(__uint_as_float(r[i]) * alpha);
                }
                continue;
              }
              __nv_bfloat16* drow =
                  reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)row * p.ldd + col0 + c;
              const __nv_bfloat16* crow =
                  p.C ? reinterpret_cast<const __nv_bfloat16*>(p.C) + (long long)row * p.ldd +
                            col0 + c
                      : nullptr;
              if (ncol >= 32 && (p.ldd & 7) == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  float v[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[8 * i + j]) * alpha;
                  if (crow) {
                    const uint4 cc = reinterpret_cast<const uint4*>(crow)[i];
                    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&cc);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      const float2 f = __bfloat1622float2(c2[j]);
                      v[2 * j] += f.x;
                      v[2 * j + 1] += f.y;
                    }
                  }
                  uint4 o;
                  o.x = pack_bf16x2(v[0], v[1]);
                  o.y = pack_bf16x2(v[2], v[3]);
                  o.z = pack_bf16x2(v[4], v[5]);
                  o.w = pack_bf16x2(v[6], v[7]);
                  reinterpret_cast<uint4*>(drow)[i] = o;
                  for (int m = 0; m < p.n_mirrors; ++m) {
                    __nv_bfloat16* mrow = reinterpret_cast<__nv_bfloat16*>(p.mirror[m]) +
                                          (long long)row * p.mirror_ld[m] + col0 + c;
                    reinterpret_cast<uint4*>(mrow)[i] = o;
                  }
                }
              } else {
                for (int i = 0; i < 32 && i < ncol; ++i) {
                  float v = __uint_as_float(r[i]) * alpha;
                  if (crow) v += __bfloat162float(crow[i]);
                  drow[i] = __float2bfloat16(v);
                  for (int m = 0; m < p.n_mirrors; ++m)
                    (reinterpret_cast<__nv_bfloat16*>(p.mirror[m]) + (long long)row * p.mirror_ld[m] + col0 + c)[i] =
                        __float2bfloat16(v);
                }
              }
            }
          }
        }
      }
      // Accumulator buffer drained: hand it back to the MMA warp.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR)
          mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[acc]), 0));
        else
          mbar_arrive(&acc_empty[acc]);
      }
      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------------------------- teardown -----
  if (*abort_word) {
    // A wait ran out.  Give copies already issued time to land before the CTA
    // (and its shared memory) goes away, then report.
    __nanosleep(200000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  // a pair leaves together: the even CTA's MMAs read the odd CTA's shared memory, and both signal each other's barriers
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    if (PAIR)
      tmem_dealloc_pair(tmem_base, kTmemCols);
    else
      tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// bf16 row-major matrix [rows, cols] with leading dimension ld (elements);
// box = box_cols x box_rows, 128-byte swizzle.
static int make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                         long long ld, int box_cols, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // First call on a thread that has no current context yet (for example an autograd worker whose first device
    // work is this launch): bind the primary context of the operand's device and encode again.
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, base) == cudaSuccess && at.device >= 0) cudaSetDevice(at.device);
    cudaFree(nullptr);
    r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS && getenv("AB_DEBUG"))
    fprintf(stderr, "cuTensorMapEncodeTiled failed: CUresult %d base %p rows %lld cols %lld ld %lld box %d x %d\n",
            (int)r, base, rows, cols, ld, box_cols, box_rows);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int A_MN, int B_MN, int EPI, int PAIR>
static int launch(const GemmMaps& maps, const GemmParams& p, int max_ctas, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, EPI, PAIR>;
  static std::atomic<unsigned long long> attr_done{0};   // one per template instantiation, one bit per device
  if (!once_per_device(attr_done, [&] {
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess;
      }))
    return -3;
  // scheduling units: CTAs, or CTA pairs (p.m_tiles then counts 256-row tiles)
  int units = p.m_tiles * p.n_tiles;
  int cap = max_ctas > 0 ? max_ctas : num_sms();
  if (PAIR) cap /= 2;
  if (cap < 1) cap = 1;
  if (units > cap) units = cap;
  if (units <= 0) return 0;
  GemmParams q = p;
  if (q.stream_k) {
    const int tiles = p.m_tiles * p.n_tiles;
    const int kb = p.k_blocks0 + p.k_blocks1;
    units = cap;
    if ((long long)tiles * kb < units) units = (int)((long long)tiles * kb);
    q.full_tiles = (tiles / units) * units;
    const long long tail_units = (long long)(tiles - q.full_tiles) * kb;
    q.units_per_cta = (tail_units + units - 1) / units;
    if (tail_units == 0) q.stream_k = 0;
  }
  if (!PAIR) {
    kern<<<units, kThreads, kSmemBytes, stream>>>(maps, q);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * units, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, maps, q) == cudaSuccess ? 0 : -4;
}

}  // namespace ab

// Operand description passed from Python: a bf16 matrix as stored in memory.
//   mn_major = 0: stored [MN, K] (reduction index contiguous)
//   mn_major = 1: stored [K, MN] (output index contiguous)
struct AbOperand {
  const void* ptr;
  long long ld;   // leading dimension in elements
  int mn_major;
};

extern "C" {

// D[M,N] = alpha * (A0*B0^T + A1*B1^T) (+ C).  Returns 0 on a successful launch.
//   epi: 0 store, 1 row statistics (vocabulary head), 2 SwiGLU (N = 2 * out)
//   k1 = 0 disables the second source.  Leading dimensions must be multiples of 8 elements and
//   base pointers 16-byte aligned (TMA); M, N and K themselves are arbitrary (tails are zero-filled).
int ab_gemm_bf16(int M, int N, int K0, int K1, const AbOperand* a0, const AbOperand* b0,
                 const AbOperand* a1, const AbOperand* b1, void* D, long long ldd, int d_is_fp32,
                 const void* C, float alpha, int epi, float* stats, float logit_scale, int* status,
                 int max_ctas, int stream_k, int n_mirrors, void* const* mirrors, const long long* mirror_lds,
                 int mirror_cols, int cta_pair,
                 void* stream) {
  using namespace ab;
  if (M <= 0 || N <= 0 || K0 <= 0 || K1 < 0) return -10;
  if (K1 > 0 && (a1->mn_major != a0->mn_major || b1->mn_major != b0->mn_major)) return -11;
  GemmMaps maps;
  auto mk = [&](CUtensorMap* m, const AbOperand* o, int mn_extent, int k_extent, int tile_mn) {
    if ((reinterpret_cast<uintptr_t>(o->ptr) & 15) || (o->ld & 7)) return -12;
    if (o->mn_major)  // memory is [K, MN]: box 64 (mn) x 64 (k)
      return make_map_bf16(m, o->ptr, k_extent, mn_extent, o->ld, 64, BK);
    return make_map_bf16(m, o->ptr, mn_extent, k_extent, o->ld, BK, tile_mn);
  };
  int rc;
  const int b_box = cta_pair ? BN / 2 : BN;   // a CTA of a pair stages half of the tile's B rows
  if ((rc = mk(&maps.a0, a0, M, K0, BM))) return rc;
  if ((rc = mk(&maps.b0, b0, N, K0, b_box))) return rc;
  if (K1 > 0) {
    if ((rc = mk(&maps.a1, a1, M, K1, BM))) return rc;
    if ((rc = mk(&maps.b1, b1, N, K1, b_box))) return rc;
  } else {
    maps.a1 = maps.a0;
    maps.b1 = maps.b0;
  }
  GemmParams p;
  p.M = M;
  p.N = N;
  p.k_blocks0 = (K0 + BK - 1) / BK;
  p.k_blocks1 = K1 > 0 ? (K1 + BK - 1) / BK : 0;
  p.m_tiles = cta_pair ? (M + 2 * BM - 1) / (2 * BM) : (M + BM - 1) / BM;
  p.n_tiles = (N + BN - 1) / BN;
  p.D = D;
  p.ldd = ldd;
  p.d_is_fp32 = d_is_fp32;
  p.C = C;
  p.alpha = alpha;
  p.stats = stats;
  p.logit_scale = logit_scale;
  p.status = status;
  p.n_mirrors = 0;
  p.mirror_cols = 0;
  if (n_mirrors > 0) {
    if (n_mirrors > 8 || epi != EPI_STORE || d_is_fp32 || stream_k) return -17;
    // scatter mode: whole 32-column chunks per destination, all of N covered, no addend
    if (mirror_cols < 0 || (mirror_cols > 0 && ((mirror_cols & 31) || (long long)mirror_cols * n_mirrors < N || C))) return -17;
    for (int m = 0; m < n_mirrors; ++m) {
      if ((reinterpret_cast<uintptr_t>(mirrors[m]) & 15) || (mirror_lds[m] & 7) || (ldd & 7)) return -17;
      p.mirror[m] = mirrors[m];
      p.mirror_ld[m] = mirror_lds[m];
    }
    p.n_mirrors = n_mirrors;
    p.mirror_cols = mirror_cols;
  }
  p.stream_k = 0;
  p.full_tiles = 0;
  p.units_per_cta = 0;
  if (stream_k) {
    // split tiles are combined in fp32: D must be fp32 and either zero-filled or accumulated in place
    if (epi != EPI_STORE || !d_is_fp32 || (C != nullptr && C != D)) return -16;
    p.stream_k = 1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int amn = a0->mn_major, bmn = b0->mn_major;
#define AB_DISPATCH(EPI, PAIR)                                                         \
  if (!amn && !bmn) return launch<0, 0, EPI, PAIR>(maps, p, max_ctas, s);              \
  if (!amn && bmn) return launch<0, 1, EPI, PAIR>(maps, p, max_ctas, s);               \
  if (amn && !bmn) return launch<1, 0, EPI, PAIR>(maps, p, max_ctas, s);               \
  return launch<1, 1, EPI, PAIR>(maps, p, max_ctas, s);
  if (epi == EPI_STORE) {
    if (cta_pair) { AB_DISPATCH(EPI_STORE, 1) }
    AB_DISPATCH(EPI_STORE, 0)
  }
  if (epi == EPI_ROWSTATS) {
    if (amn || bmn || d_is_fp32) return -13;
    if (cta_pair) return launch<0, 0, EPI_ROWSTATS, 1>(maps, p, max_ctas, s);
    return launch<0, 0, EPI_ROWSTATS, 0>(maps, p, max_ctas, s);
  }
  if (epi == EPI_SWIGLU) {
    if (amn || bmn || d_is_fp32 || (N & 1)) return -13;
    if (cta_pair) return launch<0, 0, EPI_SWIGLU, 1>(maps, p, max_ctas, s);
    return launch<0, 0, EPI_SWIGLU, 0>(maps, p, max_ctas, s);
  }
#undef AB_DISPATCH
  return -14;
}

int ab_gemm_tile_n() { return ab::BN; }

}  // extern "C"
