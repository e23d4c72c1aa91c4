// Tile schedule shared by the persistent kernel (device) and its host replay.
//
// The reference builds per-expert GEMM problems with a one-block kernel
// (csrc/fill_arguments.cuh:34-98), sorts them by k for wgrad (:80-86) and leaves
// the walk over tiles to CUTLASS' device-only group scheduler.  Here all of it is
// a few integers per CTA: an exclusive prefix sum of batch_sizes (row_start), an
// order of the experts (perm), an exclusive prefix sum of per-expert tile counts
// in that order (tile_start), and pure functions from a position in the launch
// order to (expert, rows, columns, k-range).
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

// Transposed ("swap-AB") tiles of the forward / dgrad layouts: an expert with at
// most kLightRows rows does not get a 128-row tile.  Instead 128 output COLUMNS
// ride the UMMA M dimension and the few rows ride UMMA N (a multiple of 16), so a
// 5-row expert costs an N=16 instruction instead of a padded 128 x 256 one.  Such a
// tile is kLightCols columns wide and takes kLightK of the contraction per pipeline
// stage.  (Larger experts keep 128-row tiles for their last rows too: a transposed
// tile for the remainder would sweep the expert's weights a second time.)
constexpr int kLightRows = 64;
constexpr int kLightCols = 128;
constexpr int kLightK = 128;

struct Problem {
  int mode;
  int z;
  int64_t tokens;  // rows of a
  int64_t d1;      // a.shape[1]: k for NN/NT, m for TN
  int64_t n;       // output columns
  int tile_m;      // output rows per scheduled tile: 128 (one CTA) or 256 (a CTA pair)
  int group_m;     // row-tiles swept together across the columns (L2 reuse of b)
  int light;       // 1: experts of <= kLightRows rows run as transposed tiles (NN/NT, tile_m 128)
  int order;       // 0: experts in index order.  1: experts sorted by rows, largest first
  int64_t wait_ns; // limit of every wait inside the kernel, in nanoseconds
  // Derived on the host so that decoding a tile needs no 64-bit division:
  int nt;          // column tiles of kBlockN: ceil(n / 256)
  int mt;          // TN: row tiles of c[i]: ceil(d1 / tile_m)
  int lt;          // column tiles of a transposed tile's width: ceil(n / 128)
  int wide_a;      // TN: a's columns are a multiple of 64, one TMA load brings all 64-column boxes of a stage
  int wide_b;      // TN: same for b
};

// Fills the derived fields of a Problem whose shape fields are set.
B200GMM_HD void derive(Problem* p) {
  p->nt = static_cast<int>((p->n + kBlockN - 1) / kBlockN);
  p->mt = static_cast<int>((p->d1 + p->tile_m - 1) / p->tile_m);
  p->lt = static_cast<int>((p->n + kLightCols - 1) / kLightCols);
}

struct Tile {
  int expert;
  int row0;        // NN/NT: first row of a/c (global); TN: first row of c[expert]
  int col0;        // first output column
  int valid_rows;  // rows of this tile that exist in the output
  int k_row0;      // TN: first contraction row in a/b (global); else 0
  int k_len;       // contraction length (k, or batch_sizes[expert] for TN)
  int kind;        // 0: tile_m x 256 tile; 1: transposed tile (valid_rows <= kLightRows, kLightCols columns)
};

B200GMM_HD int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

// Row-tiles of tile_m rows an expert with `rows` rows gets, and the rows that go
// to transposed tiles instead (0 if none).
B200GMM_HD int heavy_row_tiles(const Problem& p, int rows) {
  if (p.light && rows <= kLightRows) return 0;
  return ceil_div_i(rows, p.tile_m);
}
B200GMM_HD int light_rows(const Problem& p, int rows) {
  return (p.light && rows <= kLightRows) ? rows : 0;
}

// Tiles of one expert.  TN always has the full c[i] grid (empty experts still
// need their zeros written, csrc/fill_arguments.cuh:100-119).
B200GMM_HD int expert_tiles(const Problem& p, int rows) {
  if (p.mode == kTN) return p.mt * p.nt;
  return heavy_row_tiles(p, rows) * p.nt + (light_rows(p, rows) > 0 ? p.lt : 0);
}

// Pipeline stages (ring slots) one tile consumes.
B200GMM_HD int tile_stages(const Tile& t) {
  return t.kind ? (t.k_len + kLightK - 1) / kLightK : (t.k_len + kBlockK - 1) / kBlockK;
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

// `local` = tile index relative to the expert's first tile; rs/re = row_start[expert],
// row_start[expert+1] (already clamped to tokens).
B200GMM_HD Tile make_tile(const Problem& p, int expert, int local, int rs, int re) {
  Tile t;
  t.expert = expert;
  t.kind = 0;
  const int nt = p.nt;
  int mi, ni;
  if (p.mode == kTN) {
    decode_in_expert(local, p.mt, nt, p.group_m, &mi, &ni);
    t.row0 = mi * p.tile_m;
    const int left = static_cast<int>(p.d1) - t.row0;
    t.valid_rows = left < p.tile_m ? left : p.tile_m;
    t.k_row0 = rs;
    t.k_len = re - rs;
    t.col0 = ni * kBlockN;
    return t;
  }
  t.k_row0 = 0;
  t.k_len = static_cast<int>(p.d1);
  const int mt = heavy_row_tiles(p, re - rs);
  if (local < mt * nt) {
    decode_in_expert(local, mt, nt, p.group_m, &mi, &ni);
    t.row0 = rs + mi * p.tile_m;
    const int left = re - t.row0;
    t.valid_rows = left < p.tile_m ? left : p.tile_m;
    t.col0 = ni * kBlockN;
  } else {
    t.kind = 1;
    t.row0 = rs + mt * kBlockM;
    t.valid_rows = re - t.row0;
    t.col0 = (local - mt * nt) * kLightCols;
  }
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
