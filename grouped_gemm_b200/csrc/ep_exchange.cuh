// Row exchange for expert parallelism over peer memory.
//
// One kernel moves token rows between GPUs: every item is one row that is read
// from this GPU's memory and written, with plain 16-byte stores, to a row of a
// buffer on the GPU that needs it (possibly this one).  The destination
// buffers are symmetric-memory allocations mapped into this process, so the
// stores travel over NVLink / NVSwitch without a staging copy, a packing pass or
// a collective.  No TMA and no multicast is involved; remote memory is only
// ever the target of ordinary stores.
//
// The reference (tgale96/grouped_gemm) has no multi-GPU code; callers sort rows
// by expert before gmm and un-sort after.  This kernel is that permutation and
// the inter-GPU transfer in one pass.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace b200gmm {

constexpr int kPushThreads = 256;

constexpr int kPushVecsPerThread = 8;  // 16-byte loads a thread keeps in flight

// item i: row src_row[i] (or i when src_row == nullptr) of `src`
//      -> row dst_row[i] of the buffer peer_base[dst_rank[i]].
// One CTA moves one row at a time: every thread first issues all of its loads of
// the row (up to kPushVecsPerThread x 16 bytes, i.e. rows of up to 32 KiB in one
// sweep), then all of its stores, so that a whole row is in flight per CTA.
__global__ void __launch_bounds__(kPushThreads)
push_rows_kernel(const uint4* __restrict__ src, int64_t row_vecs, int64_t n_items,
                 const int32_t* __restrict__ src_row, const int32_t* __restrict__ dst_rank,
                 const int64_t* __restrict__ dst_row, void* const* __restrict__ peer_base) {
  for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int64_t sr = (src_row != nullptr) ? src_row[item] : item;
    const uint4* s = src + sr * row_vecs;
    uint4* d = static_cast<uint4*>(peer_base[dst_rank[item]]) + dst_row[item] * row_vecs;
    for (int64_t base = 0; base < row_vecs; base += int64_t(kPushVecsPerThread) * kPushThreads) {
      uint4 r[kPushVecsPerThread];
#pragma unroll
      for (int j = 0; j < kPushVecsPerThread; ++j) {
        const int64_t v = base + int64_t(j) * kPushThreads + threadIdx.x;
        if (v < row_vecs) r[j] = __ldg(s + v);
      }
#pragma unroll
      for (int j = 0; j < kPushVecsPerThread; ++j) {
        const int64_t v = base + int64_t(j) * kPushThreads + threadIdx.x;
        if (v < row_vecs) d[v] = r[j];
      }
    }
  }
}

// Top-k sum of the combine: out[t, :] = slots[t * top_k, :] + .. + slots[t * top_k +
// top_k - 1, :], added in fp32 in that order and rounded to bf16 once.  A thread owns
// 8 columns (16 bytes) of one token; all of its top_k loads are issued before the
// first add.  HBM-bound: (top_k + 1) x 2 bytes per output element.
constexpr int kSumThreads = 256;
constexpr int kSumMaxTopK = 8;

__global__ void __launch_bounds__(kSumThreads)
sum_slots_kernel(const uint4* __restrict__ slots, uint4* __restrict__ out, int64_t tokens, int top_k,
                 int64_t row_vecs) {
  const int64_t total = tokens * row_vecs;
  for (int64_t i = int64_t(blockIdx.x) * kSumThreads + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * kSumThreads) {
    const int64_t t = i / row_vecs, v = i - t * row_vecs;
    const uint4* src = slots + (t * top_k) * row_vecs + v;
    uint4 r[kSumMaxTopK];
#pragma unroll
    for (int j = 0; j < kSumMaxTopK; ++j)
      if (j < top_k) r[j] = __ldg(src + int64_t(j) * row_vecs);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll
    for (int j = 0; j < kSumMaxTopK; ++j) {
      if (j < top_k) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
    }
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) ho[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    out[i] = o;
  }
}

}  // namespace b200gmm
