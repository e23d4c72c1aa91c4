/*
 * Plain-C restatement of the reference's argument fill and of one expert's
 * product.  TEST INFRASTRUCTURE ONLY (built by oracle/Makefile into
 * oracle/libgmm_oracle.so; loaded by tests/ only).
 *
 * fill: csrc/fill_arguments.cuh:59-78 and csrc/grouped_gemm.cu:160-175 of
 * tgale96/grouped_gemm, evaluated in int64.
 * gemm: the per-expert product of grouped_gemm/ops_test.py:44-53 and
 * csrc/grouped_gemm.cu:396-435, bf16 operands, fp32 accumulation, one rounding.
 */
#include <stdint.h>
#include <string.h>

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, NaN kept quiet */
static uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* out: z rows of {m,n,k,lda,ldb,ldc,a_offset,b_offset,c_offset} */
void oracle_fill_offsets(const int64_t* batch_sizes, int z, int64_t dim_a1, int64_t n,
                         int trans_a, int trans_b, int64_t* out) {
  int64_t start = 0;
  for (int e = 0; e < z; ++e) {
    int64_t* o = out + (int64_t)e * 9;
    const int64_t size = batch_sizes[e];
    if (trans_a) {
      const int64_t m = dim_a1, k = size;
      o[0] = m; o[1] = n; o[2] = k;
      o[3] = m; o[4] = n; o[5] = n;
      o[6] = m * start; o[7] = start * n; o[8] = (int64_t)e * m * n;
    } else {
      const int64_t m = size, k = dim_a1;
      o[0] = m; o[1] = n; o[2] = k;
      o[3] = k; o[4] = trans_b ? k : n; o[5] = n;
      o[6] = start * k; o[7] = (int64_t)e * k * n; o[8] = start * n;
    }
    start += size;
  }
}

/* Grouped product on raw bf16 bit patterns, all three layouts. */
void oracle_gmm_bf16(const uint16_t* a, const uint16_t* b, uint16_t* c, const int64_t* batch_sizes,
                     int z, int64_t dim_a1, int64_t n, int trans_a, int trans_b) {
  int64_t start = 0;
  for (int e = 0; e < z; ++e) {
    const int64_t size = batch_sizes[e];
    if (trans_a) {
      const int64_t m = dim_a1;
      for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
          float acc = 0.f;
          for (int64_t r = start; r < start + size; ++r)
            acc += bf16_to_f32(a[r * m + i]) * bf16_to_f32(b[r * n + j]);
          c[((int64_t)e * m + i) * n + j] = f32_to_bf16(acc);
        }
    } else {
      const int64_t k = dim_a1;
      const uint16_t* be = b + (int64_t)e * k * n;
      for (int64_t r = start; r < start + size; ++r)
        for (int64_t j = 0; j < n; ++j) {
          float acc = 0.f;
          for (int64_t l = 0; l < k; ++l) {
            const float bv = trans_b ? bf16_to_f32(be[j * k + l]) : bf16_to_f32(be[l * n + j]);
            acc += bf16_to_f32(a[r * k + l]) * bv;
          }
          c[r * n + j] = f32_to_bf16(acc);
        }
    }
    start += size;
  }
}
