// Selected-key attention for sm_100a: every query attends its own list of key rows.
//
//   O[i, h, :] = softmax_{k in sel[i]}( scale * Q[i, h, :] . K[k, h / G, :] ) V[k, h / G, :]
//
// `sel [n_q, L]` holds key-row indices (a negative entry is an empty slot).  This is the attention of the
// sparse drafts (DSA / CSA / QSA): the indexer's top-k context tokens, compressed entries or selected blocks,
// followed by the query's own draft block.  Lists differ from query to query, so nothing can be shared between
// queries; what is shared is the key/value head: the G query heads of a group are the N dimension of the MMAs.
//
// One CTA = one query x one key/value head, tiles of 128 selected keys:
//   warps 5..8  gather the 128 K rows and 128 V rows of the tile into 128-byte-swizzled shared memory
//               (16-byte cp.async per piece, zero fill for empty slots)
//   warp 4      tcgen05.mma issuer:  S^T = Ksel Q_g^T   (M = 128 keys, N = 16 heads, K = 128)
//                                    O^T += Vsel^T P^T  (M = 128 dims, N = 16 heads, K = 128 keys)
//   warps 0..3  softmax over the key (lane) dimension: tile maxima meet in shared memory, P^T goes back as the
//               bf16 B operand, the 16 accumulator columns of O^T are rescaled when a maximum moves
// Transposed accumulators keep tensor-memory traffic at 16 columns per tile.  Two CTAs fit on an SM, so one CTA's
// gather runs under the other's softmax.
//
// Backward (same decomposition): S^T and dP^T = Vsel dO_g^T by MMA, P and dS per key lane, dQ^T += Ksel^T dS^T by
// MMA; dK / dV are rank-G updates per selected key and are added into fp32 accumulators with vector reductions
// (the same key can be selected by many queries).
//
// Every wait is bounded; a timeout sets the status word and the CTA drains and exits.
#include "common.cuh"

namespace ab {
namespace sel {

static constexpr int BK = 128;                 // selected keys per tile = TMEM lanes
static constexpr int HD = 128;                 // head dim
static constexpr int NH = 16;                  // head columns (group size padded to the MMA's minimum N)
static constexpr int kThreads = 288;
static constexpr int kTile = BK * HD * 2;      // 32 KB
static constexpr int kChunk = BK * 128;        // 16 KB: one 64-column chunk of a 128-row tile
static constexpr int kSmall = NH * HD * 2;     // 4 KB: a 16-row operand
static constexpr int kSmallChunk = NH * 128;   // 2 KB
static constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;            // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
// Meeting point of the 128 softmax threads on an mbarrier (count 128), so that this wait is bounded like every other:
// a thread that left on an abort makes the others time out instead of waiting for ever.
__device__ __forceinline__ bool group_sync(uint64_t* bar, uint32_t& uses, volatile int* abort_word) {
  mbar_arrive(bar);
  const bool ok = mbar_wait(bar, uses & 1u, abort_word);
  ++uses;
  return ok;
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Byte offset of element (row, col) in a 128-byte-swizzled K-major tile whose 64-column chunks are `chunk_bytes`
// apart (rows are 128 B; the 16-byte piece index is XORed with the row's low three bits).
__device__ __forceinline__ uint32_t swz(int row, int col, int chunk_bytes) {
  const int c = col & 63;
  return (uint32_t)((col >> 6) * chunk_bytes + row * 128 + ((((c >> 3) ^ (row & 7)) << 4) | ((c & 7) << 1)));
}

struct SelParams {
  const __nv_bfloat16* q;      // [n_q, hq, 128]
  const __nv_bfloat16* k;      // [tk, hkv, 128], row stride k_ld elements
  const __nv_bfloat16* v;
  const int* sel;              // [n_q, L]
  __nv_bfloat16* out;          // [n_q, hq, 128]        (forward: written, backward: read)
  float* lse;                  // [hq, n_q] natural log (forward: written, backward: read)
  const __nv_bfloat16* dout;   // backward
  __nv_bfloat16* dq;           // backward [n_q, hq, 128]
  float* dk;                   // backward [tk, hkv, 128] fp32, accumulated with reductions
  float* dv;
  int n_q, hq, hkv, group, tk, L;
  long long k_ld, v_ld;
  float scale, scale_log2;
  int* status;
};

// 128 producer threads copy the tile's rows of one operand: thread `pt` moves 16-byte piece pt % 16 of rows
// pt / 16 + 8 i.  Each row is 256 B in global memory and two 128-byte swizzled rows (one per chunk) in the tile.
__device__ __forceinline__ void gather_rows(uint8_t* tile, const __nv_bfloat16* src, long long ld, int kvh,
                                            const int* sel_row, int first, int L, int tk, int pt) {
  const int piece = pt & 15, r0 = pt >> 4;
  const uint32_t base = smem_u32(tile) + (piece >> 3) * kChunk;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int r = r0 + 8 * i;
    const int li = first + r;
    const int idx = li < L ? sel_row[li] : -1;
    const bool ok = idx >= 0 && idx < tk;
    const __nv_bfloat16* g = src + (ok ? (long long)idx * ld + kvh * HD + piece * 8 : 0);
    cp_async16(base + r * 128 + (((piece & 7) ^ (r & 7)) << 4), g, ok);
  }
}

// 16-row operand (the group's query heads): rows >= G are zero.  256 threads, one 16-byte piece each.
__device__ __forceinline__ void load_group_rows(uint8_t* tile, const __nv_bfloat16* rows, int G, int tid) {
  if (tid < 256) {
    const int row = tid >> 4, piece = tid & 15;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (row < G) val = reinterpret_cast<const uint4*>(rows + (size_t)row * HD)[piece];
    *reinterpret_cast<uint4*>(tile + (piece >> 3) * kSmallChunk + row * 128 + (((piece & 7) ^ (row & 7)) << 4)) = val;
  }
}

// ------------------------------------------------------------------------------------ forward ----
// TMEM: S^T [0,16)   O^T [16,32)
static constexpr int kFwdSmem = 2 * kTile + 2 * kSmall + 1024 /*barriers, reductions*/ + 1024 /*alignment*/;

__global__ void __launch_bounds__(kThreads, 2) sel_attn_fwd_kernel(const SelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTile;
  uint8_t* sQ = smem + 2 * kTile;
  uint8_t* sP = sQ + kSmall;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kSmall);
  uint64_t* k_full = bars;       // 4 arrivals (producer warps)
  uint64_t* k_free = bars + 1;   // S^T MMA of the tile retired
  uint64_t* v_full = bars + 2;   // 4
  uint64_t* v_free = bars + 3;   // P V MMA retired
  uint64_t* s_full = bars + 4;
  uint64_t* p_full = bars + 5;   // 4 arrivals (softmax warps)
  uint64_t* o_done = bars + 6;
  uint64_t* meet = bars + 7;     // 128 arrivals: the softmax threads' meeting point
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(tmem_slot + 4);   // [2][4][16]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  const int qi = blockIdx.x, kvh = blockIdx.y;
  const int n_tiles = (p.L + BK - 1) / BK;
  const int* sel_row = p.sel + (size_t)qi * p.L;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(k_full, 4); mbar_init(k_free, 1); mbar_init(v_full, 4); mbar_init(v_free, 1);
    mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(o_done, 1); mbar_init(meet, 128);
    fence_barrier_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 32); tmem_relinquish(); }
  load_group_rows(sQ, p.q + ((size_t)qi * p.hq + kvh * G) * HD, G, threadIdx.x);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp >= 5) {
    // ------------------------------------------------------------ gather producers ----
    const int pt = threadIdx.x - 160;
    for (int j = 0; j < n_tiles; ++j) {
      if (j > 0 && !mbar_wait(k_free, (j - 1) & 1, abort_word)) break;
      gather_rows(sK, p.k, p.k_ld, kvh, sel_row, j * BK, p.L, p.tk, pt);
      cp_async_wait_all();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(k_full);
      if (j > 0 && !mbar_wait(v_free, (j - 1) & 1, abort_word)) break;
      gather_rows(sV, p.v, p.v_ld, kvh, sel_row, j * BK, p.L, p.tk, pt);
      cp_async_wait_all();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(v_full);
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BK, NH, 0, 0);   // Ksel (K-major) x Q_g (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(HD, NH, 1, 0);   // Vsel^T (MN-major: dims contiguous) x P^T (K-major)
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_full, ph, abort_word)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc_mma_ss(tmem + 0, make_smem_desc(k_addr + (k >> 2) * kChunk + (k & 3) * 32, 16, 1024),
                    make_smem_desc(q_addr + (k >> 2) * kSmallChunk + (k & 3) * 32, 16, 1024), idesc_s, k ? 1u : 0u);
        tc_commit(k_free);
        tc_commit(s_full);
        if (!mbar_wait(v_full, ph, abort_word)) break;
        if (!mbar_wait(p_full, ph, abort_word)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)   // 16 keys per instruction
          tc_mma_ss(tmem + 16, make_smem_desc(v_addr + k * 2048, kChunk, 1024),
                    make_smem_desc(p_addr + (k >> 2) * kSmallChunk + (k & 3) * 32, 16, 1024), idesc_o,
                    (j | k) ? 1u : 0u);
        tc_commit(v_free);
        tc_commit(o_done);
      }
    }
  } else {
    // --------------------------------------------------------------------- softmax ----
    const int t = threadIdx.x;                                  // key slot of the tile == TMEM lane; later: output dim
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_run[NH], l_part[NH];
#pragma unroll
    for (int h = 0; h < NH; ++h) { m_run[h] = -INFINITY; l_part[h] = 0.f; }
    bool alive = true;
    uint32_t meets = 0;
    for (int j = 0; j < n_tiles && alive; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_word)) { alive = false; break; }
      tc_fence_after();
      // s_full of tile j also means P_{j-1} V_{j-1} has retired (the tensor core completes in issue order):
      // the P^T operand and the O^T accumulator may be touched now
      const int li = j * BK + t;
      const int idx = li < p.L ? sel_row[li] : -1;
      const bool ok = idx >= 0 && idx < p.tk;
      uint32_t s[NH];
      tmem_ld_32x16(tmem + lane_base + 0, s);
      tmem_ld_wait();
      float x[NH];
      float* rj = red + (j & 1) * 64;
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        x[h] = ok ? __uint_as_float(s[h]) * p.scale_log2 : -INFINITY;
        const float mx = warp_max(x[h]);
        if (lane == 0) rj[warp * NH + h] = mx;
      }
      if (!group_sync(meet, meets, abort_word)) { alive = false; break; }
      bool moved = false;
      float alpha[NH];
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        const float mt = fmaxf(fmaxf(rj[h], rj[NH + h]), fmaxf(rj[2 * NH + h], rj[3 * NH + h]));
        const float m_new = fmaxf(m_run[h], mt);
        alpha[h] = (m_new == m_run[h]) ? 1.f : fast_exp2(m_run[h] - m_new);   // m_run = -inf, m_new finite: exp2(-inf) = 0
        moved |= (alpha[h] != 1.f) && (h < G);
        const float pv = (m_new == -INFINITY) ? 0.f : fast_exp2(x[h] - m_new);
        l_part[h] = l_part[h] * alpha[h] + pv;
        m_run[h] = m_new;
        // P^T[h][key t] as bf16 into the K-major B operand (rows = heads, columns = keys of the tile)
        *reinterpret_cast<__nv_bfloat16*>(sP + swz(h, t, kSmallChunk)) = __float2bfloat16(h < G ? pv : 0.f);
      }
      if (j > 0 && moved) {   // `moved` is the same in every thread: all derive it from the shared maxima
        uint32_t o[NH];
        tmem_ld_32x16(tmem + lane_base + 16, o);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < NH; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
        tmem_st_32x16(tmem + lane_base + 16, o);
        tmem_st_wait();
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (alive && n_tiles > 0) alive = mbar_wait(o_done, (n_tiles - 1) & 1, abort_word);
    if (alive) {
      tc_fence_after();
      // row sums: every thread holds a partial over its key slots
      float* rs = red;   // [4][16]; the per-tile maxima are no longer needed
      alive = group_sync(meet, meets, abort_word);
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        const float sum = warp_sum(l_part[h]);
        if (lane == 0) rs[warp * NH + h] = sum;
      }
      alive = group_sync(meet, meets, abort_word) && alive;
    }
    if (alive) {
      const float* rs = red;
      uint32_t o[NH];
      if (n_tiles > 0) { tmem_ld_32x16(tmem + lane_base + 16, o); tmem_ld_wait(); }
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        if (h < G) {
          const float l = (rs[h] + rs[NH + h]) + (rs[2 * NH + h] + rs[3 * NH + h]);
          const int head = kvh * G + h;
          const float val = (n_tiles > 0 && l > 0.f) ? __uint_as_float(o[h]) / l : 0.f;
          p.out[((size_t)qi * p.hq + head) * HD + t] = __float2bfloat16(val);   // thread t = output dim t
          if (t == 0)
            p.lse[(size_t)head * p.n_q + qi] = l > 0.f ? (m_run[h] + log2f(l)) * 0.6931471805599453f : -INFINITY;
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
  if (warp == 4) { __syncwarp(); tmem_dealloc(tmem, 32); }
}

// ----------------------------------------------------------------------------------- backward ----
// TMEM: S^T [0,16)   dP^T [16,32)   dQ^T [32,48)
static constexpr int kBwdSmem = 2 * kTile + 3 * kSmall + 2 * NH * HD * 4 /*fp32 Q, dO*/ + 1024 + 1024;

__global__ void __launch_bounds__(kThreads, 2) sel_attn_bwd_kernel(const SelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTile;
  uint8_t* sQ = smem + 2 * kTile;
  uint8_t* sdO = sQ + kSmall;
  uint8_t* sdS = sdO + kSmall;
  float* qf = reinterpret_cast<float*>(sdS + kSmall);      // [16][128]
  float* dof = qf + NH * HD;                               // [16][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(dof + NH * HD);
  uint64_t* k_full = bars;       // 4
  uint64_t* k_free = bars + 1;   // dQ MMA retired (K is its A operand too)
  uint64_t* v_full = bars + 2;   // 4
  uint64_t* v_free = bars + 3;   // dP^T MMA retired
  uint64_t* sp_full = bars + 4;
  uint64_t* ds_full = bars + 5;  // 4
  uint64_t* dq_done = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stats = reinterpret_cast<float*>(tmem_slot + 4);  // lse2 [16], delta [16]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  const int qi = blockIdx.x, kvh = blockIdx.y;
  const int n_tiles = (p.L + BK - 1) / BK;
  const int* sel_row = p.sel + (size_t)qi * p.L;
  const size_t row0 = ((size_t)qi * p.hq + kvh * G) * HD;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(k_full, 4); mbar_init(k_free, 1); mbar_init(v_full, 4); mbar_init(v_free, 1);
    mbar_init(sp_full, 1); mbar_init(ds_full, 4); mbar_init(dq_done, 1);
    fence_barrier_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
  load_group_rows(sQ, p.q + row0, G, threadIdx.x);
  load_group_rows(sdO, p.dout + row0, G, threadIdx.x);
  // plain fp32 copies for the rank-G updates, and delta[h] = sum_d O[h, d] dO[h, d]
  for (int i = threadIdx.x; i < NH * HD; i += kThreads) {
    const int h = i >> 7;
    qf[i] = h < G ? __bfloat162float(p.q[row0 + i]) : 0.f;
    dof[i] = h < G ? __bfloat162float(p.dout[row0 + i]) : 0.f;
  }
  if (warp < 4) {
    for (int h = warp; h < NH; h += 4) {
      float acc = 0.f;
      if (h < G)
        for (int d = lane; d < HD; d += 32)
          acc += __bfloat162float(p.out[row0 + h * HD + d]) * __bfloat162float(p.dout[row0 + h * HD + d]);
      acc = warp_sum(acc);
      if (lane == 0) {
        stats[NH + h] = acc;
        float l2 = h < G ? p.lse[(size_t)(kvh * G + h) * p.n_q + qi] * kLog2e : 0.f;
        if (!(l2 > -INFINITY)) l2 = INFINITY;     // a row that saw no key: every probability is exp2(-inf) = 0
        stats[h] = l2;
      }
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp >= 5) {
    const int pt = threadIdx.x - 160;
    for (int j = 0; j < n_tiles; ++j) {
      if (j > 0 && !mbar_wait(k_free, (j - 1) & 1, abort_word)) break;
      gather_rows(sK, p.k, p.k_ld, kvh, sel_row, j * BK, p.L, p.tk, pt);
      cp_async_wait_all();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(k_full);
      if (j > 0 && !mbar_wait(v_free, (j - 1) & 1, abort_word)) break;
      gather_rows(sV, p.v, p.v_ld, kvh, sel_row, j * BK, p.L, p.tk, pt);
      cp_async_wait_all();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(v_full);
    }
  } else if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(BK, NH, 0, 0);   // rows (K-major) x group rows (K-major)
      constexpr uint32_t idesc_dq = make_idesc_bf16(HD, NH, 1, 0);   // Ksel^T (MN-major) x dS^T (K-major)
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ), do_addr = smem_u32(sdO),
                     ds_addr = smem_u32(sdS);
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_full, ph, abort_word)) break;
        if (!mbar_wait(v_full, ph, abort_word)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc_mma_ss(tmem + 0, make_smem_desc(k_addr + (k >> 2) * kChunk + (k & 3) * 32, 16, 1024),
                    make_smem_desc(q_addr + (k >> 2) * kSmallChunk + (k & 3) * 32, 16, 1024), idesc_kk, k ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc_mma_ss(tmem + 16, make_smem_desc(v_addr + (k >> 2) * kChunk + (k & 3) * 32, 16, 1024),
                    make_smem_desc(do_addr + (k >> 2) * kSmallChunk + (k & 3) * 32, 16, 1024), idesc_kk, k ? 1u : 0u);
        tc_commit(v_free);
        tc_commit(sp_full);
        if (!mbar_wait(ds_full, ph, abort_word)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          tc_mma_ss(tmem + 32, make_smem_desc(k_addr + k * 2048, kChunk, 1024),
                    make_smem_desc(ds_addr + (k >> 2) * kSmallChunk + (k & 3) * 32, 16, 1024), idesc_dq,
                    (j | k) ? 1u : 0u);
        tc_commit(k_free);
        tc_commit(dq_done);
      }
    }
  } else {
    const int t = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      if (!mbar_wait(sp_full, j & 1, abort_word)) { alive = false; break; }
      tc_fence_after();
      // sp_full of tile j also means the dQ MMA of tile j-1 has retired: dS^T may be overwritten
      const int li = j * BK + t;
      const int idx = li < p.L ? sel_row[li] : -1;
      const bool ok = idx >= 0 && idx < p.tk;
      uint32_t s[NH], dp[NH];
      tmem_ld_32x16(tmem + lane_base + 0, s);
      tmem_ld_32x16(tmem + lane_base + 16, dp);
      tmem_ld_wait();
      float pr[NH], ds[NH];
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        const bool use = ok && h < G;
        pr[h] = use ? fast_exp2(fmaf(__uint_as_float(s[h]), p.scale_log2, -stats[h])) : 0.f;
        ds[h] = pr[h] * (__uint_as_float(dp[h]) - stats[NH + h]) * p.scale;
        *reinterpret_cast<__nv_bfloat16*>(sdS + swz(h, t, kSmallChunk)) = __float2bfloat16(ds[h]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      // rank-G updates of this key's dK and dV rows (fp32 reductions: other queries select the same key)
      if (ok) {
        float* dkr = p.dk + ((size_t)idx * p.hkv + kvh) * HD;
        float* dvr = p.dv + ((size_t)idx * p.hkv + kvh) * HD;
#pragma unroll 2
        for (int d = 0; d < HD; d += 4) {
          float4 ak = make_float4(0.f, 0.f, 0.f, 0.f), av = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int h = 0; h < NH; ++h) {
            if (h < G) {
              const float4 qv = *reinterpret_cast<const float4*>(qf + h * HD + d);
              const float4 gv = *reinterpret_cast<const float4*>(dof + h * HD + d);
              ak.x = fmaf(ds[h], qv.x, ak.x); ak.y = fmaf(ds[h], qv.y, ak.y);
              ak.z = fmaf(ds[h], qv.z, ak.z); ak.w = fmaf(ds[h], qv.w, ak.w);
              av.x = fmaf(pr[h], gv.x, av.x); av.y = fmaf(pr[h], gv.y, av.y);
              av.z = fmaf(pr[h], gv.z, av.z); av.w = fmaf(pr[h], gv.w, av.w);
            }
          }
          red_add_v4(dkr + d, ak.x, ak.y, ak.z, ak.w);
          red_add_v4(dvr + d, av.x, av.y, av.z, av.w);
        }
      }
    }
    if (alive && n_tiles > 0) alive = mbar_wait(dq_done, (n_tiles - 1) & 1, abort_word);
    if (alive) {
      tc_fence_after();
      uint32_t o[NH];
      if (n_tiles > 0) { tmem_ld_32x16(tmem + lane_base + 32, o); tmem_ld_wait(); }
#pragma unroll
      for (int h = 0; h < NH; ++h)
        if (h < G)
          p.dq[row0 + h * HD + t] = __float2bfloat16(n_tiles > 0 ? __uint_as_float(o[h]) : 0.f);   // thread t = dim t
    }
  }
  if (*abort_word) {
    __nanosleep(200000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, kStatusWaitTimeout);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { __syncwarp(); tmem_dealloc(tmem, 64); }
}

static int check(const SelParams& p, int head_dim) {
  if (head_dim != HD || p.hq <= 0 || p.hkv <= 0 || p.hq % p.hkv) return -10;
  if (p.group > NH) return -11;
  if ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15) return -12;
  if ((p.k_ld & 7) || (p.v_ld & 7)) return -12;
  if (p.hkv > 65535) return -13;
  return 0;
}

}  // namespace sel
}  // namespace ab

// q / out [n_q, hq, 128] bf16 contiguous; k / v [tk, hkv, 128] bf16 with row strides k_ld / v_ld (elements);
// sel [n_q, L] int32 (negative = empty slot); lse [hq, n_q] fp32.
extern "C" int ab_sel_attn_fwd(const void* q, const void* k, const void* v, const int* sel, void* out, float* lse,
                               int n_q, int tk, int L, int hq, int hkv, int head_dim, long long k_ld, long long v_ld,
                               float scale, int* status, void* stream) {
  using namespace ab;
  using namespace ab::sel;
  SelParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k = reinterpret_cast<const __nv_bfloat16*>(k);
  p.v = reinterpret_cast<const __nv_bfloat16*>(v);
  p.sel = sel;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.n_q = n_q; p.hq = hq; p.hkv = hkv; p.group = hkv > 0 ? hq / hkv : 0; p.tk = tk; p.L = L;
  p.k_ld = k_ld; p.v_ld = v_ld;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.status = status;
  if (int rc = check(p, head_dim)) return rc;
  if (n_q <= 0) return 0;
  static std::atomic<unsigned long long> attr_done{0};
  if (!once_per_device(attr_done, [&] {
        return cudaFuncSetAttribute(sel_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem) == cudaSuccess;
      }))
    return -3;
  sel_attn_fwd_kernel<<<dim3(n_q, hkv), kThreads, kFwdSmem, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// dq [n_q, hq, 128] bf16 is written; dk / dv [tk, hkv, 128] fp32 must be zeroed by the caller and receive sums.
extern "C" int ab_sel_attn_bwd(const void* q, const void* k, const void* v, const int* sel, const void* out,
                               const float* lse, const void* dout, void* dq, float* dk, float* dv, int n_q, int tk, int L,
                               int hq, int hkv, int head_dim, long long k_ld, long long v_ld, float scale, int* status,
                               void* stream) {
  using namespace ab;
  using namespace ab::sel;
  SelParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k = reinterpret_cast<const __nv_bfloat16*>(k);
  p.v = reinterpret_cast<const __nv_bfloat16*>(v);
  p.sel = sel;
  p.out = const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(out));
  p.lse = const_cast<float*>(lse);
  p.dout = reinterpret_cast<const __nv_bfloat16*>(dout);
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk = dk; p.dv = dv;
  p.n_q = n_q; p.hq = hq; p.hkv = hkv; p.group = hkv > 0 ? hq / hkv : 0; p.tk = tk; p.L = L;
  p.k_ld = k_ld; p.v_ld = v_ld;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.status = status;
  if (int rc = check(p, head_dim)) return rc;
  if (n_q <= 0) return 0;
  static std::atomic<unsigned long long> attr_done{0};
  if (!once_per_device(attr_done, [&] {
        return cudaFuncSetAttribute(sel_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem) == cudaSuccess;
      }))
    return -3;
  sel_attn_bwd_kernel<<<dim3(n_q, hkv), kThreads, kBwdSmem, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
