// Host-side planners of the grouped GEMM: fill the tile and segment tables that the kernel walks
// (csrc/grouped_gemm_sm100.cu).  One call per launch; a few microseconds for hundreds of problems, where the
// same arithmetic in array-library calls costs a few hundred.  The reference has no counterpart: it loops over
// experts in Python (aspec/models/draft/ling_moe.py:101-115).
#include <algorithm>
#include <cstdint>
#include <vector>

namespace {

constexpr int BM = 128, BN = 256, BK = 64;

struct GTile {
  uint64_t d;
  int64_t ldd;
  int32_t rows, cols, seg0, nseg;
};
struct GSeg {
  int32_t a_map, a_mn, a_k, b_map, b_mn, b_k, k_blocks, pad;
};
static_assert(sizeof(GTile) == 32 && sizeof(GSeg) == 32, "table layout is shared with the kernel");

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace

extern "C" {

// Number of tiles (= segments) of a row-problem list; problems with rows <= 0 are skipped.
int64_t ab_plan_rows_count(int n_problems, const int64_t* rows, int64_t N) {
  int64_t total = 0;
  const int64_t n_tiles = ceil_div(N, BN);
  for (int i = 0; i < n_problems; ++i)
    if (rows[i] > 0) total += ceil_div(rows[i], BM) * n_tiles;
  return total;
}

// D_i[rows_i, N] = A_{src_i}[a_row_i : a_row_i + rows_i, :K] * W_{expert_i}^T, stored at out_base[dst_i] + out_row_i.
// Tiles of a problem are ordered n-tile major so that CTAs in flight share weight tiles.  b_t: the stacked weights
// are [E, K, N] (MN-major B), else [E, N, K].  Returns the number of tiles written.
int64_t ab_plan_rows_gemm(int n_problems, const int64_t* src, const int64_t* a_row, const int64_t* rows,
                          const int64_t* expert, const int64_t* dst, const int64_t* out_row, const uint64_t* out_base,
                          const int64_t* out_ld, int elem_size, int64_t N, int64_t K, int b_map, int b_t, void* tiles_out,
                          void* segs_out) {
  GTile* tiles = static_cast<GTile*>(tiles_out);
  GSeg* segs = static_cast<GSeg*>(segs_out);
  const int64_t n_tiles = ceil_div(N, BN);
  const int32_t k_blocks = static_cast<int32_t>(ceil_div(K, BK));
  int64_t t = 0;
  for (int i = 0; i < n_problems; ++i) {
    if (rows[i] <= 0) continue;
    const int64_t m_tiles = ceil_div(rows[i], BM);
    const int64_t ld = out_ld[dst[i]];
    for (int64_t nt = 0; nt < n_tiles; ++nt) {
      for (int64_t mt = 0; mt < m_tiles; ++mt, ++t) {
        GTile& tile = tiles[t];
        tile.d = out_base[dst[i]] + static_cast<uint64_t>(((out_row[i] + mt * BM) * ld + nt * BN) * elem_size);
        tile.ldd = ld;
        tile.rows = static_cast<int32_t>(std::min<int64_t>(BM, rows[i] - mt * BM));
        tile.cols = static_cast<int32_t>(std::min<int64_t>(BN, N - nt * BN));
        tile.seg0 = static_cast<int32_t>(t);
        tile.nseg = 1;
        GSeg& sg = segs[t];
        sg.a_map = static_cast<int32_t>(src[i]);
        sg.a_mn = static_cast<int32_t>(a_row[i] + mt * BM);
        sg.a_k = 0;
        sg.b_map = b_map;
        sg.b_mn = static_cast<int32_t>(b_t ? nt * BN : expert[i] * N + nt * BN);
        sg.b_k = static_cast<int32_t>(b_t ? expert[i] * K : 0);
        sg.k_blocks = k_blocks;
        sg.pad = 0;
      }
    }
  }
  return t;
}

// out[e][Ma, Nb] = sum over runs i with expert_i == e of A_i^T B_i (both operands MN-major, reduction over rows).
// Runs must be sorted by expert (stable).  n_tiles_out = E * tiles per matrix; returns the number of segments.
int64_t ab_plan_wgrad_gemm(int n_runs, const int64_t* expert, const int64_t* a_src, const int64_t* a_row,
                           const int64_t* b_src, const int64_t* b_row, const int64_t* rows, int n_experts, int64_t Ma,
                           int64_t Nb, uint64_t out_base, int64_t out_stride_e, int64_t out_ld, int elem_size, int b_map0,
                           void* tiles_out, void* segs_out) {
  GTile* tiles = static_cast<GTile*>(tiles_out);
  GSeg* segs = static_cast<GSeg*>(segs_out);
  const int64_t m_tiles = ceil_div(Ma, BM), n_tiles = ceil_div(Nb, BN);
  std::vector<int> first(n_experts + 1, 0);
  for (int i = 0; i < n_runs; ++i) first[expert[i] + 1]++;
  for (int e = 0; e < n_experts; ++e) first[e + 1] += first[e];
  int64_t t = 0, s = 0;
  for (int e = 0; e < n_experts; ++e) {
    const int run0 = first[e], run1 = first[e + 1];
    for (int64_t nt = 0; nt < n_tiles; ++nt) {
      for (int64_t mt = 0; mt < m_tiles; ++mt, ++t) {
        GTile& tile = tiles[t];
        tile.d = out_base + static_cast<uint64_t>((e * out_stride_e + mt * BM * out_ld + nt * BN) * elem_size);
        tile.ldd = out_ld;
        tile.rows = static_cast<int32_t>(std::min<int64_t>(BM, Ma - mt * BM));
        tile.cols = static_cast<int32_t>(std::min<int64_t>(BN, Nb - nt * BN));
        tile.seg0 = static_cast<int32_t>(s);
        tile.nseg = run1 - run0;
        for (int r = run0; r < run1; ++r, ++s) {
          GSeg& sg = segs[s];
          sg.a_map = static_cast<int32_t>(a_src[r]);
          sg.a_mn = static_cast<int32_t>(mt * BM);
          sg.a_k = static_cast<int32_t>(a_row[r]);
          sg.b_map = static_cast<int32_t>(b_map0 + b_src[r]);
          sg.b_mn = static_cast<int32_t>(nt * BN);
          sg.b_k = static_cast<int32_t>(b_row[r]);
          sg.k_blocks = static_cast<int32_t>(ceil_div(rows[r], BK));
          sg.pad = 0;
        }
      }
    }
  }
  return s;
}

}  // extern "C"
