// Memory-bound fused kernels for sm_100a: RMSNorm, per-head QK-norm + RoPE,
// SwiGLU, the vocabulary-sized loss / gradient pass of the DSpark, DFlash and
// EAGLE objectives, and the flat-buffer optimizer step (grad norm, clip, AdamW,
// bf16 write-back).  All of them stream each operand once or twice with
// 128-bit accesses and keep statistics in fp32.
#include "common.cuh"

namespace ab {

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// Block-wide sum / max over up to 1024 threads; result broadcast to all threads.
template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = (lane < nw) ? scratch[lane] : (IS_MAX ? -INFINITY : 0.f);
  r = IS_MAX ? warp_max(r) : warp_sum(r);
  return r;
}

// ------------------------------------------------------------- RMSNorm ------
// One CTA per row; H % 8 == 0.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   float* __restrict__ rstd_out, int rows, int H, float eps) {
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
  const int nv = H >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_reduce<false>(ss, scratch);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8], g[8];
    unpack8(xr[i], f);
    unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
    yr[i] = pack8(f);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat));  dw[h] += sum_rows dy*xhat  (fp32 atomics).
// Persistent: each CTA walks rows blockIdx.x, +gridDim.x, ... and keeps its dw partial in
// registers (thread t owns vectors t, t+blockDim, ...; at most 4 vectors => H <= 8*4*blockDim).
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w,
                                   const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw, int rows, int H) {
  __shared__ float scratch[32];
  const int nv = H >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float acc[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[a][j] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * H);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float fx[8], fd[8], fw[8];
      unpack8(xr[i], fx);
      unpack8(dyr[i], fd);
      unpack8(wr[i], fw);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += fd[j] * fw[j] * fx[j] * rstd;
    }
    dot = block_reduce<false>(dot, scratch) / H;
    int a = 0;
    for (int i = threadIdx.x; i < nv; i += blockDim.x, ++a) {
      float fx[8], fd[8], fw[8], o[8];
      unpack8(xr[i], fx);
      unpack8(dyr[i], fd);
      unpack8(wr[i], fw);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = fx[j] * rstd;
        o[j] = rstd * (fd[j] * fw[j] - xh * dot);
        if (a < 4) acc[a][j] += fd[j] * xh;
      }
      dxr[i] = pack8(o);
    }
  }
  int a = 0;
  for (int i = threadIdx.x; i < nv && a < 4; i += blockDim.x, ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dw + i * 8 + j, acc[a][j]);
}

// ------------------------------------------------- QK-norm + RoPE -----------
// x [N, H, D] bf16; one warp per (n, h) row; D in {64,128,256}: each lane holds E = D/32
// consecutive elements; the rotate-half partner (i +- D/2) sits in lane ^ 16.
template <int D>
__global__ void qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                        const __nv_bfloat16* __restrict__ w,
                                        const int* __restrict__ pos,
                                        const float* __restrict__ inv_freq,
                                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                        long long n_rows, int H, float eps, float scaling) {
  constexpr int E = D / 32;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  float wv[E];
#pragma unroll
  for (int e = 0; e < E; ++e) wv[e] = w ? __bfloat162float(w[lane * E + e]) : 1.f;
  for (long long r = warp0; r < n_rows; r += nwarps) {
    const __nv_bfloat16* xr = x + r * D;
    float v[E];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      v[e] = __bfloat162float(xr[lane * E + e]);
      ss += v[e] * v[e];
    }
    ss = warp_sum(ss);
    const float rstd = w ? rsqrtf(ss / D + eps) : 1.f;
    if (lane == 0 && rstd_out) rstd_out[r] = rstd;
    const int p = pos[r / H];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float xn = v[e] * rstd * wv[e];
      const float other = __shfl_xor_sync(0xffffffffu, xn, 16);
      const int i = lane * E + e;
      const int fi = i < D / 2 ? i : i - D / 2;
      float s, c;
      sincosf((float)p * inv_freq[fi], &s, &c);
      s *= scaling;
      c *= scaling;
      // first half: x1*c - x2*s ; second half: x2*c + x1*s
      const float out = i < D / 2 ? xn * c - other * s : xn * c + other * s;
      y[r * D + i] = __float2bfloat16(out);
    }
  }
}

// Backward: dxn = R^T dy; dx = rstd*(dxn*w - xhat*mean(dxn*w*xhat)); dw += dxn*xhat.
template <int D>
__global__ void qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                        const __nv_bfloat16* __restrict__ x,
                                        const __nv_bfloat16* __restrict__ w,
                                        const int* __restrict__ pos,
                                        const float* __restrict__ inv_freq,
                                        const float* __restrict__ rstd_in,
                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                        long long n_rows, int H, float scaling) {
  constexpr int E = D / 32;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  float wv[E], acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    wv[e] = w ? __bfloat162float(w[lane * E + e]) : 1.f;
    acc[e] = 0.f;
  }
  for (long long r = warp0; r < n_rows; r += nwarps) {
    const int p = pos[r / H];
    const float rstd = w ? rstd_in[r] : 1.f;
    float g[E], xh[E];
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int i = lane * E + e;
      const float d = __bfloat162float(dy[r * D + i]);
      const float other = __shfl_xor_sync(0xffffffffu, d, 16);
      const int fi = i < D / 2 ? i : i - D / 2;
      float s, c;
      sincosf((float)p * inv_freq[fi], &s, &c);
      s *= scaling;
      c *= scaling;
      // transpose of the rotation: first half d1*c + d2*s ; second half d2*c - d1*s
      g[e] = i < D / 2 ? d * c + other * s : d * c - other * s;
      xh[e] = __bfloat162float(x[r * D + i]) * rstd;
      dot += g[e] * wv[e] * xh[e];
    }
    if (w) {
      dot = warp_sum(dot) / D;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        acc[e] += g[e] * xh[e];
        dx[r * D + lane * E + e] = __float2bfloat16(rstd * (g[e] * wv[e] - xh[e] * dot));
      }
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) dx[r * D + lane * E + e] = __float2bfloat16(g[e]);
    }
  }
  if (w && dw) {
    // combine the block's warps in shared memory first: one atomic per column per CTA
    __shared__ float red[D];
    for (int i = threadIdx.x; i < D; i += blockDim.x) red[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int e = 0; e < E; ++e) atomicAdd(&red[lane * E + e], acc[e]);
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(dw + i, red[i]);
  }
}

// --------------------------------------------------------------- SwiGLU -----
// gu [R, 2I] with gate in [0,I) and up in [I,2I); act [R, I].  clamp > 0 applies the Ling
// limits (gate <= clamp, |up| <= clamp) before the product.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                  long long R, int I, float clamp) {
  const long long nv = R * (I >> 3);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nv;
       v += (long long)gridDim.x * blockDim.x) {
    const long long r = v / (I >> 3);
    const int c = (int)(v - r * (I >> 3)) << 3;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + c), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gg = g[j], uu = u[j];
      if (clamp > 0.f) {
        gg = fminf(gg, clamp);
        uu = fminf(fmaxf(uu, -clamp), clamp);
      }
      o[j] = gg / (1.f + __expf(-gg)) * uu;
    }
    *reinterpret_cast<uint4*>(act + r * I + c) = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgu, long long R, int I, float clamp) {
  const long long nv = R * (I >> 3);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nv;
       v += (long long)gridDim.x * blockDim.x) {
    const long long r = v / (I >> 3);
    const int c = (int)(v - r * (I >> 3)) << 3;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + c), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c), u);
    unpack8(*reinterpret_cast<const uint4*>(dact + r * I + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gg = g[j], uu = u[j];
      bool g_live = true, u_live = true;
      if (clamp > 0.f) {
        g_live = gg <= clamp;
        u_live = fabsf(uu) <= clamp;
        gg = fminf(gg, clamp);
        uu = fminf(fmaxf(uu, -clamp), clamp);
      }
      const float sg = 1.f / (1.f + __expf(-gg));
      const float silu = gg * sg;
      dg[j] = g_live ? d[j] * uu * (sg + silu * (1.f - sg)) : 0.f;
      du[j] = u_live ? d[j] * silu : 0.f;
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + c) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + I + c) = pack8(du);
  }
}

// ------------------------------------------------- softmax partial merge ----
// stats [n_tiles, M, 2] (max, sumexp) -> lse [M]
__global__ void merge_rowstats_kernel(const float2* __restrict__ stats, float* __restrict__ lse,
                                      int n_tiles, int M) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= M) return;
  float m = -INFINITY;
  for (int t = 0; t < n_tiles; ++t) m = fmaxf(m, stats[(size_t)t * M + r].x);
  float s = 0.f;
  for (int t = 0; t < n_tiles; ++t) {
    const float2 v = stats[(size_t)t * M + r];
    if (v.x > -INFINITY) s += v.y * __expf(v.x - m);
  }
  lse[r] = m + __logf(s);
}

// ----------------------------------------- vocabulary loss + gradient -------
// One CTA per supervised row r.
//   s = logits[r, :] (student, bf16), normaliser lse_s[r]
//   t = teacher[t_index[r], :] (bf16), normaliser lse_t[t_index[r]]   (may be absent)
//   p = softmax(s), q = softmax(t)
// mode 0 (DSpark / DFlash):  loss = a_ce * CE(s, label) + a_l1 * sum|p - q|
// mode 1 (EAGLE forward KL): loss = lse_s - sum_v q_v s_v          (soft-target cross entropy)
// Outputs per row: ce, l1 (or kl), correct (argmax(s) == label), and the gradient
//   dlogits[r, :] = weight[r] * d loss / d s     written over `logits` in place (bf16).
// Rows with weight 0 still get their statistics; their gradient row is zero.
struct VocabLossParams {
  __nv_bfloat16* logits;        // [R, ld]
  const __nv_bfloat16* teacher; // [Tt, ld_t] or null
  const float* lse_s;           // [R]
  const float* lse_t;           // [Tt]
  const int* t_index;           // [R] or null (identity)
  const long long* labels;      // [R]
  const float* weight;          // [R] loss weight of the row (decay * eval)
  float* ce_out;                // [R]
  float* l1_out;                // [R]
  float* correct_out;           // [R]
  long long ld, ld_t;
  int V;
  int mode;
  float a_ce, a_l1;
  int write_grad;
  // vocabulary shards (all null / 0 for the unsharded head):
  //   partial == 1: statistics pass over this rank's columns only; lse_s / lse_t are the GLOBAL normalisers;
  //                 ce_out = -s[label] when the label's column is local else 0, l1_out = partial sum|p - q|,
  //                 c_io = partial sum p*sign(p - q), best_val / best_idx = local arg-max (global column index).
  //   partial == 2: gradient pass only; c_io holds the sum of all ranks' partials.
  int partial;
  long long vocab_offset;       // global index of local column 0
  float* c_io;                  // [R]
  float* best_val_out;          // [R]
  int* best_idx_out;            // [R]
};

__global__ void __launch_bounds__(512) vocab_loss_kernel(const VocabLossParams p) {
  __shared__ float scratch[32];
  __shared__ int iscratch[32];
  const int r = blockIdx.x;
  __nv_bfloat16* srow = p.logits + (size_t)r * p.ld;
  const int ti = p.t_index ? p.t_index[r] : r;
  const __nv_bfloat16* trow = p.teacher ? p.teacher + (size_t)ti * p.ld_t : nullptr;
  const float ls = p.lse_s[r];
  const float lt = trow ? p.lse_t[ti] : 0.f;
  const long long label = p.labels[r] - p.vocab_offset;   // local column of the label (may be out of range)
  const float wgt = p.weight[r];
  const int nv = p.V >> 3;  // V % 8 == 0 is required by the launcher
  constexpr float L2E = 1.4426950408889634f;
  float l1 = 0.f, c = 0.f, cross = 0.f, best = -INFINITY, tbest = -INFINITY;
  int best_i = 0x7fffffff, tbest_i = 0x7fffffff;
  if (p.partial == 2) {
    c = p.c_io[r];
  } else {
  // pass A: l1 = sum|p-q|, c = sum p*sign(p-q), cross = sum q*s, argmax
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float s[8], t[8];
    unpack8(reinterpret_cast<const uint4*>(srow)[i], s);
    if (trow) unpack8(reinterpret_cast<const uint4*>(trow)[i], t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s[j] > best) {
        best = s[j];
        best_i = i * 8 + j;
      }
      if (trow && p.mode == 1 && t[j] > tbest) {
        tbest = t[j];
        tbest_i = i * 8 + j;
      }
      if (trow) {
        const float pp = fast_exp2((s[j] - ls) * L2E);
        const float qq = fast_exp2((t[j] - lt) * L2E);
        const float d = pp - qq;
        l1 += fabsf(d);
        c += d > 0.f ? pp : (d < 0.f ? -pp : 0.f);
        cross += qq * s[j];
      }
    }
  }
  l1 = block_reduce<false>(l1, scratch);
  c = block_reduce<false>(c, scratch);
  cross = block_reduce<false>(cross, scratch);
  // argmax: max value, then smallest index holding it
  const float gbest = block_reduce<true>(best, scratch);
  int cand = (best == gbest) ? best_i : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) iscratch[threadIdx.x >> 5] = cand;
  __syncthreads();
  int gidx = 0x7fffffff;
  for (int wi = 0; wi < (int)(blockDim.x >> 5); ++wi) gidx = min(gidx, iscratch[wi]);
  int tidx = 0x7fffffff;
  if (p.mode == 1 && trow) {   // arg-max of the teacher row (EAGLE accuracy compares the two arg-maxima)
    const float gt = block_reduce<true>(tbest, scratch);
    int tc = (tbest == gt) ? tbest_i : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tc = min(tc, __shfl_xor_sync(0xffffffffu, tc, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) iscratch[threadIdx.x >> 5] = tc;
    __syncthreads();
    for (int wi = 0; wi < (int)(blockDim.x >> 5); ++wi) tidx = min(tidx, iscratch[wi]);
  }

  const float s_label = (label >= 0 && label < p.V) ? __bfloat162float(srow[label]) : 0.f;
  if (threadIdx.x == 0) {
    if (p.partial == 1) {
      p.ce_out[r] = -s_label;
      p.l1_out[r] = l1;
      p.c_io[r] = c;
      p.best_val_out[r] = gbest;
      p.best_idx_out[r] = (int)p.vocab_offset + gidx;
    } else {
      p.ce_out[r] = p.mode == 1 ? (ls - cross) : (ls - s_label);
      p.l1_out[r] = l1;
      p.correct_out[r] = (gidx == (p.mode == 1 && trow ? tidx : (int)label)) ? 1.f : 0.f;
    }
  }
  }  // statistics pass
  if (!p.write_grad) return;
  __syncthreads();
  // pass B: gradient
  const float gce = wgt * p.a_ce, gl1 = wgt * p.a_l1;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float s[8], t[8], g[8];
    unpack8(reinterpret_cast<const uint4*>(srow)[i], s);
    if (trow) unpack8(reinterpret_cast<const uint4*>(trow)[i], t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float pp = fast_exp2((s[j] - ls) * L2E);
      float gj;
      if (p.mode == 1) {
        const float qq = fast_exp2((t[j] - lt) * L2E);
        gj = wgt * (pp - qq);
      } else {
        gj = gce * pp;
        if (i * 8 + j == (int)label) gj -= gce;
        if (trow && gl1 != 0.f) {
          const float qq = fast_exp2((t[j] - lt) * L2E);
          const float d = pp - qq;
          const float sg = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
          gj += gl1 * pp * (sg - c);
        }
      }
      g[j] = gj;
    }
    reinterpret_cast<uint4*>(srow)[i] = pack8(g);
  }
}

// ------------------------------------------------------- optimizer ----------
// sum of squares of an fp32 buffer -> out[0] (fp32 atomics); out[1] counts non-finite values.
__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float scratch[32];
  float ss = 0.f, bad = 0.f;
  const long long n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = g4[i];
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    if (!isfinite(v.x) || !isfinite(v.y) || !isfinite(v.z) || !isfinite(v.w)) bad = 1.f;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n4 << 2; i < n; ++i) {
      ss += g[i] * g[i];
      if (!isfinite(g[i])) bad = 1.f;
    }
  ss = block_reduce<false>(ss, scratch);
  bad = block_reduce<true>(bad, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(out, ss);
    if (bad > 0.f) atomicAdd(out + 1, 1.f);
  }
}

// Fused AdamW over flat buffers.  ctrl (device, fp32):
//   ctrl[0] = sum of squares of all gradients (already reduced over ranks)
//   ctrl[1] = non-finite count (> 0 => skip the step entirely)
//   ctrl[2] = gradient pre-scale (loss-denominator normalisation), applied before clipping
//   ctrl[4] = number of APPLIED updates including this one (device-side step counter: a skipped update does not
//             advance Adam's bias correction); read when the host passes bc1 <= 0, else bc1 / bc2 are used as given
// clip coefficient = min(1, max_norm / (pre_scale * sqrt(ctrl[0]) + 1e-6)).
__global__ void adamw_kernel(float* __restrict__ master, const float* __restrict__ grad,
                             float* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ param, long long n,
                             const float* __restrict__ ctrl, float lr, float beta1, float beta2,
                             float eps, float wd, float bc1, float bc2, float max_norm) {
  if (ctrl[1] > 0.f || !isfinite(ctrl[0])) return;
  if (bc1 <= 0.f) {
    const float t = fmaxf(ctrl[4], 1.f);
    bc1 = 1.f - powf(beta1, t);
    bc2 = 1.f - powf(beta2, t);
  }
  const float pre = ctrl[2];
  const float norm = pre * sqrtf(ctrl[0]);
  float coef = pre;
  if (max_norm > 0.f) coef *= fminf(1.f, max_norm / (norm + 1e-6f));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float g = grad[i] * coef;
    float w = master[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    w = w * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    master[i] = w;
    param[i] = __float2bfloat16(w);
  }
}

// bf16 buffer *= fp32 device scalar (gradient rescale without a host sync).
__global__ void scale_bf16_kernel(__nv_bfloat16* __restrict__ x, long long n,
                                  const float* __restrict__ scalar) {
  const float s = *scalar;
  const long long nv = n >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<uint4*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= s;
    reinterpret_cast<uint4*>(x)[i] = pack8(f);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nv << 3; i < n; ++i) x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
}

// out_bf16[i] = in_fp32[i] * scalar  (used after split-K fp32 accumulation)
__global__ void cast_scale_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                  long long n, const float* __restrict__ scalar, float mult) {
  const float s = (scalar ? *scalar : 1.f) * mult;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i] * s);
}

static inline int grid_for(long long work, int block, int cap = 148 * 8) {
  long long g = (work + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace ab

extern "C" {
using namespace ab;
#define STREAM reinterpret_cast<cudaStream_t>(stream)
#define LAUNCH_OK (cudaGetLastError() == cudaSuccess ? 0 : -4)

int ab_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int H, float eps,
                   void* stream) {
  if (H & 7) return -10;
  if (rows <= 0) return 0;
  const int block = H >= 2048 ? 256 : 128;
  rmsnorm_fwd_kernel<<<rows, block, 0, STREAM>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                 (__nv_bfloat16*)y, rstd, rows, H, eps);
  return LAUNCH_OK;
}
// dw (fp32 [H]) must be zero-initialised (or hold a running sum) by the caller.
int ab_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                   float* dw, int rows, int H, void* stream) {
  if (H & 7) return -10;
  if (rows <= 0) return 0;
  int block = 256;
  while (8 * 4 * block < H && block < 1024) block <<= 1;
  if (8 * 4 * block < H) return -11;
  const int grid = rows < 148 ? rows : 148;   // persistent: one dw flush (H atomics) per CTA
  rmsnorm_bwd_kernel<<<grid, block, 0, STREAM>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                 (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx,
                                                 dw, rows, H);
  return LAUNCH_OK;
}
int ab_qk_norm_rope_fwd(const void* x, const void* w, const int* pos, const float* inv_freq, void* y,
                        float* rstd, long long N, int H, int D, float eps, float scaling,
                        void* stream) {
  const long long rows = N * H;
  if (rows <= 0) return 0;
  const int grid = grid_for(rows, 8);
#define QKF(DD)                                                                                    \
  qk_norm_rope_fwd_kernel<DD><<<grid, 256, 0, STREAM>>>((const __nv_bfloat16*)x,                   \
                                                        (const __nv_bfloat16*)w, pos, inv_freq,     \
                                                        (__nv_bfloat16*)y, rstd, rows, H, eps,      \
                                                        scaling)
  if (D == 64) QKF(64);
  else if (D == 128) QKF(128);
  else if (D == 256) QKF(256);
  else return -10;
#undef QKF
  return LAUNCH_OK;
}
int ab_qk_norm_rope_bwd(const void* dy, const void* x, const void* w, const int* pos,
                        const float* inv_freq, const float* rstd, void* dx, float* dw, long long N,
                        int H, int D, float scaling, void* stream) {
  const long long rows = N * H;
  if (rows <= 0) return 0;
  const int grid = grid_for(rows, 8, 148 * 2);
#define QKB(DD)                                                                                    \
  qk_norm_rope_bwd_kernel<DD><<<grid, 256, 0, STREAM>>>(                                           \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, pos, inv_freq,   \
      rstd, (__nv_bfloat16*)dx, dw, rows, H, scaling)
  if (D == 64) QKB(64);
  else if (D == 128) QKB(128);
  else if (D == 256) QKB(256);
  else return -10;
#undef QKB
  return LAUNCH_OK;
}
int ab_swiglu_fwd(const void* gu, void* act, long long R, int I, float clamp, void* stream) {
  if (I & 7) return -10;
  if (R <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(R * (I >> 3), 256), 256, 0, STREAM>>>((const __nv_bfloat16*)gu,
                                                                     (__nv_bfloat16*)act, R, I, clamp);
  return LAUNCH_OK;
}
int ab_swiglu_bwd(const void* gu, const void* dact, void* dgu, long long R, int I, float clamp,
                  void* stream) {
  if (I & 7) return -10;
  if (R <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(R * (I >> 3), 256), 256, 0, STREAM>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dact, (__nv_bfloat16*)dgu, R, I, clamp);
  return LAUNCH_OK;
}
int ab_merge_rowstats(const float* stats, float* lse, int n_tiles, int M, void* stream) {
  if (M <= 0) return 0;
  merge_rowstats_kernel<<<(M + 127) / 128, 128, 0, STREAM>>>((const float2*)stats, lse, n_tiles, M);
  return LAUNCH_OK;
}
int ab_vocab_loss(void* logits, const void* teacher, const float* lse_s, const float* lse_t,
                  const int* t_index, const long long* labels, const float* weight, float* ce_out,
                  float* l1_out, float* correct_out, long long ld, long long ld_t, int R, int V,
                  int mode, float a_ce, float a_l1, int write_grad, void* stream) {
  if ((V & 7) || (ld & 7) || (ld_t & 7)) return -10;
  if (R <= 0) return 0;
  VocabLossParams p;
  p.logits = (__nv_bfloat16*)logits;
  p.teacher = (const __nv_bfloat16*)teacher;
  p.lse_s = lse_s;
  p.lse_t = lse_t;
  p.t_index = t_index;
  p.labels = labels;
  p.weight = weight;
  p.ce_out = ce_out;
  p.l1_out = l1_out;
  p.correct_out = correct_out;
  p.ld = ld;
  p.ld_t = ld_t;
  p.V = V;
  p.mode = mode;
  p.a_ce = a_ce;
  p.a_l1 = a_l1;
  p.write_grad = write_grad;
  p.partial = 0;
  p.vocab_offset = 0;
  p.c_io = nullptr;
  p.best_val_out = nullptr;
  p.best_idx_out = nullptr;
  vocab_loss_kernel<<<R, 512, 0, STREAM>>>(p);
  return LAUNCH_OK;
}
// Vocabulary-sharded form of the same kernel (mode 0).  phase 1 = statistics over the local columns, phase 2 =
// gradient with the globally summed `c`.  `lse_s` / `lse_t` are the normalisers over the FULL vocabulary.
int ab_vocab_loss_shard(void* logits, const void* teacher, const float* lse_s, const float* lse_t,
                        const int* t_index, const long long* labels, const float* weight, float* ce_part,
                        float* l1_part, float* c_io, float* best_val, int* best_idx, long long ld,
                        long long ld_t, int R, int V_local, long long vocab_offset, float a_ce, float a_l1,
                        int phase, void* stream) {
  if ((V_local & 7) || (ld & 7) || (ld_t & 7) || (phase != 1 && phase != 2)) return -10;
  if (R <= 0) return 0;
  VocabLossParams p;
  p.logits = (__nv_bfloat16*)logits;
  p.teacher = (const __nv_bfloat16*)teacher;
  p.lse_s = lse_s;
  p.lse_t = lse_t;
  p.t_index = t_index;
  p.labels = labels;
  p.weight = weight;
  p.ce_out = ce_part;
  p.l1_out = l1_part;
  p.correct_out = nullptr;
  p.ld = ld;
  p.ld_t = ld_t;
  p.V = V_local;
  p.mode = 0;
  p.a_ce = a_ce;
  p.a_l1 = a_l1;
  p.write_grad = phase == 2;
  p.partial = phase;
  p.vocab_offset = vocab_offset;
  p.c_io = c_io;
  p.best_val_out = best_val;
  p.best_idx_out = best_idx;
  vocab_loss_kernel<<<R, 512, 0, STREAM>>>(p);
  return LAUNCH_OK;
}
int ab_sumsq(const float* g, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for((n + 3) / 4, 256, 148 * 4), 256, 0, STREAM>>>(g, n, out);
  return LAUNCH_OK;
}
int ab_adamw(float* master, const float* grad, float* m, float* v, void* param, long long n,
             const float* ctrl, float lr, float beta1, float beta2, float eps, float wd, float bc1,
             float bc2, float max_norm, void* stream) {
  if (n <= 0) return 0;
  adamw_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, STREAM>>>(master, grad, m, v, (__nv_bfloat16*)param,
                                                              n, ctrl, lr, beta1, beta2, eps, wd, bc1,
                                                              bc2, max_norm);
  return LAUNCH_OK;
}
int ab_scale_bf16(void* x, long long n, const float* scalar, void* stream) {
  if (n <= 0) return 0;
  scale_bf16_kernel<<<grid_for((n + 7) / 8, 256), 256, 0, STREAM>>>((__nv_bfloat16*)x, n, scalar);
  return LAUNCH_OK;
}
int ab_cast_scale(const float* in, void* out, long long n, const float* scalar, float mult,
                  void* stream) {
  if (n <= 0) return 0;
  cast_scale_kernel<<<grid_for(n, 256), 256, 0, STREAM>>>(in, (__nv_bfloat16*)out, n, scalar, mult);
  return LAUNCH_OK;
}
}  // extern "C"
