// Tile schedule shared by the persistent kernel (device) and its host replay.
//
// The reference builds per-expert GEMM problems with a one-block kernel
// (csrc/fill_arguments.cuh:34-98) and leaves the walk over tiles to CUTLASS'
// device-only group scheduler.  Here both jobs are a few integers per CTA:
// an exclusive prefix sum of batch_sizes (row_start), an exclusive prefix sum
// of per-expert tile counts (tile_start), and a pure function from a global tile
// index to (expert, rows, columns, k-range).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define B200GMM_HD __host__ __device__ __forceinline__
#else
#define B200GMM_HD inline
#endif

namespace b200gmm {

enum Mode : int {
  kNN = 0,  // c[rows_i] = a[rows_i] @ b[i]       (forward)
  kNT = 1,  // c[rows_i] = a[rows_i] @ b[i]^T     (dgrad, or forward with trans_b)
  kTN = 2,  // c[i]      = a[rows_i]^T @ b[rows_i] (wgrad)
};

constexpr int kBlockM = 128;  // output rows per CTA (UMMA M per CTA)
constexpr int kBlockN = 256;  // output tile cols   (UMMA N)
constexpr int kBlockK = 64;   // k depth per pipeline stage = one 128-byte swizzle row of bf16

struct Problem {
  int mode;
  int z;
  int64_t tokens;  // rows of a
  int64_t d1;      // a.shape[1]: k for NN/NT, m for TN
  int64_t n;       // output columns
  int tile_m;      // output rows per scheduled tile: 128 (one CTA) or 256 (a CTA pair)
  int group_m;     // row-tiles swept together across the columns (L2 reuse of b)
  int direct_store;  // 1: epilogue writes every row with plain stores (no TMA stores)
};

struct Tile {
  int expert;
  int row0;        // NN/NT: first row of a/c (global); TN: first row of c[expert]
  int col0;        // first output column
  int valid_rows;  // rows of this tile (of tile_m) that exist in the output
  int k_row0;      // TN: first contraction row in a/b (global); else 0
  int k_len;       // contraction length (k, or batch_sizes[expert] for TN)
};

B200GMM_HD int ceil_div_i(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

B200GMM_HD int col_tiles(const Problem& p) { return ceil_div_i(p.n, kBlockN); }

// Tiles of one expert.  TN always has the full c[i] grid (empty experts still
// need their zeros written, csrc/fill_arguments.cuh:100-119).
B200GMM_HD int expert_tiles(const Problem& p, int64_t rows) {
  const int nt = col_tiles(p);
  if (p.mode == kTN) return ceil_div_i(p.d1, p.tile_m) * nt;
  return ceil_div_i(rows, p.tile_m) * nt;
}

// Within one expert: walk group_m row-tiles down, then step one column-tile
// right, so that concurrently running CTAs share a and b panels in L2.
B200GMM_HD void decode_in_expert(int local, int row_tiles, int nt, int group_m, int* mi, int* ni) {
  const int group_span = group_m * nt;
  const int g = local / group_span;
  const int first = g * group_m;
  const int gm = (row_tiles - first) < group_m ? (row_tiles - first) : group_m;
  const int r = local - g * group_span;
  *mi = first + r % gm;
  *ni = r / gm;
}

// `local` = tile index relative to tile_start[expert]; rs/re = row_start[expert],
// row_start[expert+1] (already clamped to tokens).
B200GMM_HD Tile make_tile(const Problem& p, int expert, int local, int rs, int re) {
  Tile t;
  t.expert = expert;
  const int nt = col_tiles(p);
  int mi, ni;
  if (p.mode == kTN) {
    const int mt = ceil_div_i(p.d1, p.tile_m);
    decode_in_expert(local, mt, nt, p.group_m, &mi, &ni);
    t.row0 = mi * p.tile_m;
    const int left = static_cast<int>(p.d1) - t.row0;
    t.valid_rows = left < p.tile_m ? left : p.tile_m;
    t.k_row0 = rs;
    t.k_len = re - rs;
  } else {
    const int mt = ceil_div_i(re - rs, p.tile_m);
    decode_in_expert(local, mt, nt, p.group_m, &mi, &ni);
    t.row0 = rs + mi * p.tile_m;
    const int left = re - t.row0;
    t.valid_rows = left < p.tile_m ? left : p.tile_m;
    t.k_row0 = 0;
    t.k_len = static_cast<int>(p.d1);
  }
  t.col0 = ni * kBlockN;
  return t;
}

// The nine per-expert values of the reference's GemmProblem
// (csrc/fill_arguments.cuh:13-18, :66-78), in int64.  `start` is the exclusive
// prefix sum of batch_sizes at expert `e`, `size` is batch_sizes[e].
B200GMM_HD void fill_fields(const Problem& p, int e, int64_t start, int64_t size, int64_t* out9) {
  if (p.mode == kTN) {
    const int64_t m = p.d1, n = p.n, k = size;
    out9[0] = m; out9[1] = n; out9[2] = k;
    out9[3] = m;  // a is read as column-major m x k: leading dimension = rows
    out9[4] = n; out9[5] = n;
    out9[6] = m * start; out9[7] = start * n; out9[8] = static_cast<int64_t>(e) * m * n;
  } else {
    const int64_t m = size, n = p.n, k = p.d1;
    out9[0] = m; out9[1] = n; out9[2] = k;
    out9[3] = k;
    out9[4] = (p.mode == kNT) ? k : n;  // NT reads b[i] as column-major k x n
    out9[5] = n;
    out9[6] = start * k; out9[7] = static_cast<int64_t>(e) * k * n; out9[8] = start * n;
  }
}

}  // namespace b200gmm
