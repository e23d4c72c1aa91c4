// The persistent grouped-GEMM kernel for sm_100a.
//
// One CTA per SM works through the output tiles of all experts (schedule.cuh).
// Inside a CTA three roles run concurrently:
//   warp 0      TMA producer: fills a ring of {A tile, B tile} stages in shared
//               memory (128-byte swizzle), one mbarrier per stage;
//   warp 1      MMA issuer: one lane issues tcgen05.mma (bf16 x bf16 -> fp32 in
//               TMEM), commits each stage back to the producer and each finished
//               accumulator to the epilogue; two 256-column accumulators alternate
//               so the epilogue of tile i overlaps the main loop of tile i+1;
//   warps 2-9   epilogue: each warp owns 32 rows x 128 columns of the tile (TMEM
//               lane quadrant = warp % 4, column half = (warp - 2) / 4).  It
//               tcgen05.ld's 32 columns at a time (the next load is in flight while
//               the current one is converted), rounds to bf16, stages the 32x32
//               chunk in swizzled shared memory and writes it with a TMA tensor
//               store; a warp whose 32 rows do not all exist (ragged last tile of
//               an expert) stores its valid rows directly;
//   warp 10     scheduler (leader CTA): draws tile positions from a global counter,
//               several tiles ahead of the other roles, and hands them over through
//               a small ring in shared memory (in both CTAs of a pair); for wgrad
//               it also prepares, ahead of time, the tensor maps clipped to the
//               expert a tile belongs to.
//
// Two variants, chosen on the host:
//   CTAS == 1   every CTA owns 128 x 256 output tiles (4 stages of 48 KiB).  The
//               last <= 64 rows of an expert run as a transposed tile instead: 128
//               output columns on UMMA M, the rows on UMMA N (schedule.cuh);
//   CTAS == 2   a pair of CTAs (a 2-CTA cluster on neighbouring SMs) owns
//               256 x 256 tiles: each CTA stages its own 128 rows of A and HALF of
//               the B tile, and the leader's tcgen05.mma.cta_group::2 reads both
//               halves.  That cuts the L2 -> shared-memory traffic per flop by a
//               third and shrinks a stage to 32 KiB, so six stages fit.  No TMA
//               multicast is used anywhere.
//
// Optional template variants:
//   GATHER      row i of A is row a_rows[i] of another tensor: one extra warp per
//               ring stage fetches the rows with cp.async in place of the TMA box
//               loads of A (B still comes by TMA); also for wgrad, where the
//               gathered rows are the contraction;
//   SWIGLU      (forward / dgrad layouts) two right operands; the accumulator holds
//               128 gate and 128 up columns and the epilogue writes silu(gate) * up.
// and run-time options of the epilogue: rows scattered to addresses given per row
// (row_dest), scaled per row (row_scale) and added to the destination instead of
// stored (reduce_add).
//
// This replaces the CUTLASS GemmGrouped instantiations of the reference
// (csrc/grouped_gemm.cu:38-81, :324-371), its argument-fill kernel
// (csrc/fill_arguments.cuh:34-98) and the k==0 zero-fill kernels
// (csrc/fill_arguments.cuh:100-131) with a single launch.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx.cuh"
#include "schedule.cuh"

namespace b200gmm {

constexpr int kEpilogueWarps = 8;
constexpr int kSchedWarp = 2 + kEpilogueWarps;        // warp 10
constexpr int kThreads = 32 * (kSchedWarp + 1);       // 352
constexpr int kMaxExperts = 1024;
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxStages = 6;
constexpr uint32_t kBoxBytes = 64 * kBlockK * 2;  // one 64-wide MN-major TMA box: 8 KiB
// wgrad keeps private, editable copies of its two tensor maps in the caller's
// workspace: kMapSlots {a, b} pairs per cluster, edited in turn.  The scheduler
// edits a slot only when every tile that used it has all its loads landed (the
// MMA warp counts finished tiles).
constexpr int kMapSlots = 8;
constexpr int kMaxCtas = 256;  // workspace is sized for this many CTAs
// Ring through which the scheduler hands tile positions to the other roles.  Deep
// enough that the producer can run ahead by a ring of one-stage tiles plus both
// accumulators, and that the scheduler's own latencies (the counter's round trip,
// a tensor-map edit) stay hidden behind tiles already handed out.
constexpr int kSchedSlots = 8;

// wgrad gives up ring stages for larger epilogue staging: its tiles can be a single
// k-block deep (few rows per expert, or none), and then the kernel runs at the
// speed of its output stores.  Each epilogue warp has two buffers of 32 rows x 64
// columns there (128-byte rows), used in turn, so that a warp fills one while
// the TMA store of the other still reads; the forward / dgrad layouts have one
// buffer of 32 x 32 per warp.
template <int CTAS, int MODE = kNN>
struct Geometry {
  static constexpr int kStages = (MODE == kTN) ? ((CTAS == 1) ? 3 : 4) : ((CTAS == 1) ? 4 : 6);
  static constexpr int kOutBufs = (MODE == kTN) ? 2 : 1;  // staging buffers per epilogue warp
  static constexpr uint32_t kOutBufBytes = (MODE == kTN) ? 4096u : 2048u;
  static constexpr int kBCols = kBlockN / CTAS;                 // B columns staged by one CTA
  static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;    // 16 KiB
  static constexpr uint32_t kBBytes = kBCols * kBlockK * 2;     // 32 or 16 KiB
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStages * kStageBytes;  // 192 KiB (wgrad: 128 or 144 KiB)
  static constexpr uint32_t kOutBytes = kEpilogueWarps * kOutBufs * kOutBufBytes;  // 16 KiB (wgrad: 64 KiB)
};

// A transposed tile's stage inside a one-CTA ring slot: 128 columns x 128 k of the
// weights (32 KiB: two k-halves of 16 KiB) followed by up to 64 rows x 128 k of
// the activations (two k-halves of 8 KiB).
constexpr uint32_t kLightWBytes = kLightCols * kLightK * 2;        // 32 KiB
constexpr uint32_t kLightWHalf = kLightWBytes / 2;                 // 16 KiB per 64 of k
constexpr uint32_t kLightXHalf = kLightRows * kBlockK * 2;         // 8 KiB per 64 of k
constexpr uint32_t kLightXBox = 32 * kBlockK * 2;                  // one 32-row TMA box: 4 KiB
static_assert(kLightWBytes + 2 * kLightXHalf <= Geometry<1>::kStageBytes, "a transposed stage must fit a ring slot");

// The gather variant adds one warp per ring stage; each fetches the rows of A for
// the k-blocks that land in its stage.
template <int CTAS, int MODE = kNN>
constexpr int gather_threads() { return kThreads + 32 * Geometry<CTAS, MODE>::kStages; }

// The push variant adds four warps that move rows between GPUs while the tensor
// cores work (in the default, bulk-copy form of the transfer only one of their
// threads is busy): the dispatch that has to precede the NEXT product (e.g. the
// gradient rows the dgrad product will need, sent while the forward product runs)
// rides inside this launch instead of being a pass of its own.  The rows are
// independent of the product: item i is row src_row[i] (or i) of `src` -> row
// dst_row[i] of the buffer peer_base[dst_rank[i]], exactly what push_rows_kernel
// moves.  No multicast; remote memory is only written.
constexpr int kPushWarps = 4;
constexpr int kGemmPushThreads = kThreads + 32 * kPushWarps;
constexpr int kPushVecsInFlight = 8;  // 16-byte loads a lane keeps in flight

struct PushArgs {
  const uint4* src;          // nullptr: nothing to push
  int64_t row_vecs;          // 16-byte pieces per row
  int64_t n_items;
  const int32_t* src_row;    // may be nullptr (item i reads row i)
  const int32_t* dst_rank;
  const int64_t* dst_row;
  void* const* peer_base;
  int64_t interval_ns;       // a push warp starts its j-th item no earlier than j * interval_ns after its first (0: no pacing)
  int via_tma;               // 1: rows travel global -> shared -> peer as bulk async copies issued by one thread
};
// Staging of the bulk-copy form of the transfer: three chunks in flight per thread block.
constexpr uint32_t kPushChunkBytes = 2048;
constexpr int kPushChunks = 3;
constexpr uint32_t kPushStageBytes = kPushChunkBytes * kPushChunks;


struct __align__(8) SmemTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sched_full[kSchedSlots];
  uint64_t sched_empty[kSchedSlots];
  int sched_tile[kSchedSlots];      // position of the launch order
  int sched_map[kSchedSlots];       // wgrad: map slot of the tile (bit 30: freshly edited), else 0
  uint32_t tiles_done;              // tiles of this cluster whose loads have all landed
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t handoff_fault;           // a role was handed a position out of order (self-check of the ring)
  uint32_t role_sum[16];            // per taking warp: count of positions taken (low 8 bits) + 256 * their sum
  uint64_t push_full[4];            // push variant, bulk-copy form: a staged chunk has landed (kPushChunks used)
  int row_start[kMaxExperts + 1];   // exclusive prefix sum of batch_sizes, by expert
  int tile_start[kMaxExperts + 1];  // exclusive prefix sum of tile counts, by position in perm
  uint16_t perm[kMaxExperts];       // expert at each position of the launch order
};

// One size for every instantiation: the largest layout (forward / dgrad).
constexpr size_t kSmemBytes =
    1024 /*alignment slack*/ + Geometry<1>::kRingBytes + Geometry<1>::kOutBytes + sizeof(SmemTail);
static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
// The push variant's staging chunks follow the tail (forward / dgrad layouts only).
constexpr size_t kPushStageOffset = (sizeof(SmemTail) + 127) / 128 * 128;
constexpr size_t kSmemBytesPush = kSmemBytes - sizeof(SmemTail) + kPushStageOffset + kPushStageBytes;
static_assert(kSmemBytesPush <= 232448, "the push variant's staging must fit too");
static_assert(Geometry<1>::kRingBytes == Geometry<2>::kRingBytes, "both variants use the same ring size");
static_assert(Geometry<1, kTN>::kRingBytes + Geometry<1, kTN>::kOutBytes <= Geometry<1>::kRingBytes + Geometry<1>::kOutBytes &&
              Geometry<2, kTN>::kRingBytes + Geometry<2, kTN>::kOutBytes <= Geometry<1>::kRingBytes + Geometry<1>::kOutBytes,
              "the wgrad layout must fit the common size");

// Inclusive prefix sum across the warp.
template <typename T>
__device__ __forceinline__ T warp_inclusive_scan(T v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const T up = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += up;
  }
  return v;
}

// One step of the exclusive prefix sum of batch_sizes: the 32 experts base ..
// base + 31 (zeros past z), added to the running carry.  Returns this lane's
// exclusive sum and advances the carry.  The scan every kernel of this library
// runs, whether it feeds the tile schedule or the exported argument fill.
__device__ __forceinline__ int64_t scan_step(int64_t v, int lane, int64_t* carry) {
  const int64_t incl = warp_inclusive_scan(v, lane);
  const int64_t start = *carry + incl - v;
  *carry += __shfl_sync(0xffffffffu, incl, 31);
  return start;
}

// The schedule of one launch, built in shared memory by every CTA for itself
// (all threads of the CTA must call this; it synchronises them):
//   row_start   exclusive prefix sums of batch_sizes (int64 arithmetic, 32 experts
//               per step with a running carry); rows are clamped to `tokens` so
//               that a bad batch_sizes can never push a store out of bounds;
//   perm        the experts in launch order: by index, or (order == 1) by number
//               of rows, largest first, ties by index (the reference sorts its
//               wgrad problems the same way, csrc/fill_arguments.cuh:80-86), so
//               that the launch ends on the shortest tiles;
//   tile_start  exclusive prefix sums of the per-expert tile counts in that order.
__device__ __forceinline__ void build_schedule(const Problem& p, const int64_t* __restrict__ batch_sizes,
                                               SmemTail* tail, uint32_t* status) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int scan_warp = (blockDim.x >= 96) ? 2 : 0;
  int* row_start = tail->row_start;
  if (warp == scan_warp) {
    int64_t carry = 0;
    uint32_t flags = 0;
    for (int base = 0; base < p.z; base += 32) {
      const int e = base + lane;
      int64_t v = (e < p.z) ? batch_sizes[e] : 0;
      if (v < 0) { v = 0; flags |= 0x2u; }
      int64_t start = scan_step(v, lane, &carry);
      if (start + v > p.tokens) flags |= 0x4u;
      if (start > p.tokens) start = p.tokens;
      if (e < p.z) row_start[e] = static_cast<int>(start);
    }
    if (lane == 0) row_start[p.z] = static_cast<int>(carry < p.tokens ? carry : p.tokens);
    flags = __reduce_or_sync(0xffffffffu, flags);
    if (flags != 0u && lane == 0 && status != nullptr && blockIdx.x == 0) atomicOr(status, flags);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.z; e += blockDim.x) {
    int rank = e;
    if (p.order) {
      const int mine = row_start[e + 1] - row_start[e];
      rank = 0;
      int prev = row_start[0];
      for (int j = 0; j < p.z; ++j) {
        const int next = row_start[j + 1];
        const int rj = next - prev;
        prev = next;
        rank += (rj > mine) ? 1 : 0;
        rank += (rj == mine && j < e) ? 1 : 0;
      }
    }
    tail->perm[rank] = static_cast<uint16_t>(e);
  }
  __syncthreads();
  if (warp == scan_warp) {
    int carry = 0;
    for (int base = 0; base < p.z; base += 32) {
      const int pos = base + lane;
      int tiles = 0;
      if (pos < p.z) {
        const int e = tail->perm[pos];
        tiles = expert_tiles(p, row_start[e + 1] - row_start[e]);
      }
      const int incl = warp_inclusive_scan(tiles, lane);
      if (pos < p.z) tail->tile_start[pos] = carry + incl - tiles;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) tail->tile_start[p.z] = carry;
  }
}

// Position of the launch order -> tile.  Every role keeps its own copy; positions
// arrive in increasing order, so the expert cursor only ever moves forward.
struct TileWalker {
  const Problem& p;
  const SmemTail* tail;
  int total;
  int pos;
  __device__ TileWalker(const Problem& p_, const SmemTail* tail_)
      : p(p_), tail(tail_), total(tail_->tile_start[p_.z]), pos(0) {}
  __device__ __forceinline__ bool decode(int t, Tile* out) {
    if (t < 0 || t >= total) return false;
    while (t >= tail->tile_start[pos + 1]) ++pos;
    const int e = tail->perm[pos];
    *out = make_tile(p, e, t - tail->tile_start[pos], tail->row_start[e], tail->row_start[e + 1]);
    return true;
  }
};

// Where a role's tile positions come from: the leader CTA's scheduler thread
// publishes each position (and, for wgrad, the tile's map slot) through
// sched_tile / sched_map / sched_full, in its own CTA and in its peer; every other
// role takes them from there and releases the slot on the leader's sched_empty.
constexpr int kNoTile = -1;  // a wait was abandoned
constexpr int kMapFresh = 1 << 30;  // sched_map flag: the slot was edited for this tile

template <bool kPair>
struct TileFeed {
  SmemTail* tail;
  ptx::WaitCtx wait;
  uint32_t taken;   // positions taken (or published) so far
  int map;          // sched_map entry of the position taken last
  bool remote;      // this role sits in the peer CTA: what it reads was written from the leader
  int last;         // position taken last (-1: none yet)
  uint32_t sum;     // sum of the positions taken

  __device__ TileFeed(SmemTail* tail_, const ptx::WaitCtx& w, bool in_peer = false)
      : tail(tail_), wait(w), taken(0), map(0), remote(in_peer), last(-1), sum(0) {}

  // Leaves this role's tally for the teardown check: every taking role of a CTA
  // must have been handed the same positions.
  __device__ __forceinline__ void tally(int warp) {
    tail->role_sum[warp & 15] = (taken & 0xffu) + (sum << 8);
  }

  // Consumer side, called by every lane of a warp (warp_wide) or by one thread.
  __device__ __forceinline__ int take(bool warp_wide, int lane) {
    const uint32_t slot = taken % kSchedSlots;
    const uint32_t parity = (taken / kSchedSlots) & 1u;
    ++taken;
    const uint32_t full = ptx::smem_u32(&tail->sched_full[slot]);
    const bool got = (kPair && remote) ? ptx::mbar_wait<true, 32>(full, parity, wait)
                                       : ptx::mbar_wait<false, 32>(full, parity, wait);
    if (!got) return kNoTile;
    const int t = *reinterpret_cast<volatile int*>(&tail->sched_tile[slot]);
    map = *reinterpret_cast<volatile int*>(&tail->sched_map[slot]);
    // Self-check of the hand-off: positions reach every role in strictly
    // increasing order.  One that does not is never used: the fault is recorded,
    // the launch is told to drain, and this role stops (warp-uniformly).
    bool bad = (t <= last);
    if (warp_wide) bad = __any_sync(0xffffffffu, bad);
    if (bad) {
      tail->handoff_fault = 1u;
      *wait.abort_flag = 1u;
      return kNoTile;
    }
    last = t;
    sum += static_cast<uint32_t>(t);
    if (warp_wide) __syncwarp();
    if (!warp_wide || lane == 0) {
      // Both values are in registers: the slot may be overwritten from here on.
      const uint32_t bar = ptx::smem_u32(&tail->sched_empty[slot]);
      if (kPair) ptx::mbar_arrive_cluster(ptx::mapa(bar, 0));
      else ptx::mbar_arrive(bar);
    }
    return t;
  }

  // Scheduler side (one thread of the leader CTA): hand position t to everyone.
  __device__ __forceinline__ bool publish(int t, int map_entry) {
    const uint32_t slot = taken % kSchedSlots;
    const uint32_t parity = (taken / kSchedSlots) & 1u;
    ++taken;
    if (!ptx::mbar_wait<kPair, 0>(ptx::smem_u32(&tail->sched_empty[slot]), parity ^ 1u, wait)) return false;
    *reinterpret_cast<volatile int*>(&tail->sched_tile[slot]) = t;
    *reinterpret_cast<volatile int*>(&tail->sched_map[slot]) = map_entry;
    ptx::mbar_arrive(ptx::smem_u32(&tail->sched_full[slot]));
    if (kPair) {
      ptx::st_shared_cluster_u32(ptx::mapa(ptx::smem_u32(&tail->sched_tile[slot]), 1), static_cast<uint32_t>(t));
      ptx::st_shared_cluster_u32(ptx::mapa(ptx::smem_u32(&tail->sched_map[slot]), 1), static_cast<uint32_t>(map_entry));
      ptx::mbar_arrive_release_cluster(ptx::mapa(ptx::smem_u32(&tail->sched_full[slot]), 1));
    }
    return true;
  }
};

template <int MODE, int CTAS, bool GATHER = false, bool SWIGLU = false, bool PUSH = false>
__global__ void __launch_bounds__(GATHER ? gather_threads<CTAS, MODE>() : (PUSH ? kGemmPushThreads : kThreads), 1)
gmm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
           const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_c,
           const __grid_constant__ CUtensorMap map_a2, __nv_bfloat16* __restrict__ c,
           const int64_t* __restrict__ batch_sizes, const Problem p,
           uint32_t* status, CUtensorMap* map_slots, uint32_t* sched_counter, const int64_t* __restrict__ row_dest,
           const int32_t* __restrict__ a_rows, const __nv_bfloat16* __restrict__ a_src,
           const int64_t a_src_rows, const float* __restrict__ row_scale, const int reduce_add,
           const int64_t dest_lo, const int64_t dest_hi, const __nv_bfloat16* __restrict__ gate_grad,
           const PushArgs push) {
  static_assert(!SWIGLU || MODE != kTN, "the gated product is a forward product");
  static_assert(!PUSH || (!GATHER && !SWIGLU && MODE != kTN), "push warps exist in the plain forward / dgrad kernels");
  // SWIGLU: two right operands of n columns each, b (gate) and b2 (up).  The
  // schedule runs over 2n virtual columns, 256 per tile: accumulator columns
  // [0,128) are a @ b[:, c0 .. c0+128), columns [128,256) are a @ b2[:, c0 ..
  // c0+128) with c0 = col0 / 2, and the epilogue writes the 128 output columns
  // silu(gate) * up.
  using G = Geometry<CTAS, MODE>;
  constexpr int kStages = G::kStages;
  constexpr bool kPair = (CTAS == 2);
  // Transposed tiles exist in the plain one-CTA forward / dgrad kernels only
  // (map_a2: the activations with 32-row boxes; NT also uses map_b2: b with
  // 128-row boxes).
  constexpr bool kLight = (MODE != kTN) && (CTAS == 1) && !GATHER && !SWIGLU;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;  // 1024-byte aligned: required by the 128-byte swizzle
  const uint32_t stage_base = raw_addr + pad;
  const uint32_t out_base = stage_base + G::kRingBytes;
  SmemTail* tail = reinterpret_cast<SmemTail*>(smem + G::kRingBytes + G::kOutBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;  // 0 = leader (issues the MMAs)
  const bool leader = (cta_rank == 0u);
  const ptx::WaitCtx wait{&tail->abort_flag, static_cast<uint64_t>(p.wait_ns)};

  // ------------------------------------------------------------ prologue
  if (warp == 0) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_a);
      ptx::prefetch_tensormap(&map_b);
      if (SWIGLU || (kLight && MODE == kNT)) ptx::prefetch_tensormap(&map_b2);
      if (kLight) ptx::prefetch_tensormap(&map_a2);
      ptx::prefetch_tensormap(&map_c);
      for (int s = 0; s < kStages; ++s) {
        // the producer's expect_tx arrival, plus one arrival by the gather warp that owns
        // this stage in each CTA
        ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1 + (GATHER ? CTAS : 0));
        ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 1);
      }
      for (int i = 0; i < 2; ++i) {
        ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[i]), 1);
        ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[i]), kEpilogueWarps * CTAS);
      }
      // Takers of a published tile position: per CTA the producer thread, the epilogue
      // warps and the gather warps, plus the leader's MMA warp.
      constexpr uint32_t kTakers = CTAS * (1 + kEpilogueWarps + (GATHER ? kStages : 0)) + 1;
      for (int i = 0; i < kSchedSlots; ++i) {
        ptx::mbar_init(ptx::smem_u32(&tail->sched_full[i]), 1);
        ptx::mbar_init(ptx::smem_u32(&tail->sched_empty[i]), kTakers);
      }
      tail->tiles_done = 0u;
      tail->abort_flag = 0u;
      tail->handoff_fault = 0u;
      for (int i = 0; i < 16; ++i) tail->role_sum[i] = 0xffffffffu;
      if (PUSH)
        for (int i = 0; i < kPushChunks; ++i) ptx::mbar_init(ptx::smem_u32(&tail->push_full[i]), 1);
      ptx::fence_mbar_init();
    }
    __syncwarp();
  } else if (warp == 1) {
    if (kPair) {
      ptx::tmem_alloc_pair(ptx::smem_u32(&tail->tmem_base), kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(&tail->tmem_base), kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  build_schedule(p, batch_sizes, tail, status);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (kPair) ptx::cluster_sync();  // the peer's barriers exist before anything arrives on them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tail->tmem_base;

  constexpr bool kAMn = (MODE == kTN);                 // A operand MN-major (wgrad reads a^T)
  constexpr bool kBMn = (MODE == kNN || MODE == kTN);  // B operand MN-major
  constexpr uint32_t kIdesc =
      ptx::make_idesc_bf16(kBlockM * CTAS, kBlockN, kAMn ? 1 : 0, kBMn ? 1 : 0);

  const int first_tile = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const int tile_stride = kPair ? (gridDim.x >> 1) : gridDim.x;
  const int row_off = static_cast<int>(cta_rank) * kBlockM;  // this CTA's rows inside a pair tile
  const int col_off = static_cast<int>(cta_rank) * G::kBCols;  // this CTA's share of the B tile

  // wgrad: the editable copies of the two tensor maps, one set per cluster (both
  // CTAs of a pair load through the same copies).
  CUtensorMap* my_maps = map_slots + size_t(first_tile) * (kMapSlots * 2);

  if (warp == 0) {
    // ---------------------------------------------------------- TMA producer
    if (lane == 0) {
      TileWalker walk(p, tail);
      TileFeed<kPair> feed(tail, wait, !leader);
      Tile t;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      // Bytes this CTA's TMA loads bring per stage: the gather warps fetch A themselves.
      constexpr uint32_t kTmaBytes = GATHER ? G::kBBytes : G::kStageBytes;
      const CUtensorMap* tn_a = my_maps;
      const CUtensorMap* tn_b = my_maps + 1;
      while (ok) {
        const int pos = feed.take(false, 0);
        if (pos == kNoTile) { ok = false; break; }
        if (!walk.decode(pos, &t)) break;
        const int nkb = tile_stages(t);
        if (kLight && t.kind) {
          // Transposed tile: per stage 128 columns x 128 k of b[expert] (the UMMA A
          // operand) and the tile's rows x 128 k of a (the UMMA B operand, K-major,
          // fetched in boxes of 32 rows; rows past the tile's last are never stored).
          const int row_boxes = (t.valid_rows + 31) >> 5;
          const uint32_t bytes = kLightWBytes + 2u * uint32_t(row_boxes) * kLightXBox;
          for (int kb = 0; kb < nkb; ++kb) {
            if (!ptx::mbar_wait(ptx::smem_u32(&tail->empty[s]), ph ^ 1u, wait)) { ok = false; break; }
            const uint32_t bar = ptx::smem_u32(&tail->full[s]);
            const uint32_t sw = stage_base + s * G::kStageBytes;
            const uint32_t sx = sw + kLightWBytes;
            ptx::mbar_arrive_expect_tx(bar, bytes);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int k0 = kb * kLightK + h * kBlockK;
              if (MODE == kNN) {
                ptx::tma_load_3d(sw + h * kLightWHalf, &map_b, bar, t.col0, k0, t.expert);
                ptx::tma_load_3d(sw + h * kLightWHalf + kBoxBytes, &map_b, bar, t.col0 + 64, k0, t.expert);
              } else {
                ptx::tma_load_3d(sw + h * kLightWHalf, &map_b2, bar, k0, t.col0, t.expert);
              }
              for (int i = 0; i < row_boxes; ++i)
                ptx::tma_load_2d(sx + h * kLightXHalf + i * kLightXBox, &map_a2, bar, k0, t.row0 + i * 32);
            }
            if (++s == kStages) { s = 0; ph ^= 1u; }
          }
          continue;
        }
        if (MODE == kTN && nkb > 0) {
          // The scheduler clipped a copy of both maps at this expert's last row, so
          // that the rows a k-block would read from the next expert are out of bounds
          // for TMA and arrive as zeros.  A freshly edited copy has to be acquired by
          // the thread that loads through it.
          tn_a = my_maps + (feed.map & (kMapSlots - 1)) * 2;
          tn_b = tn_a + 1;
          if (feed.map & kMapFresh) {
            ptx::fence_tensormap_acquire(tn_a);
            ptx::fence_tensormap_acquire(tn_b);
          }
        }
        for (int kb = 0; kb < nkb; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&tail->empty[s]), ph ^ 1u, wait)) { ok = false; break; }
          const uint32_t local_bar = ptx::smem_u32(&tail->full[s]);
          const uint32_t sa = stage_base + s * G::kStageBytes;
          const uint32_t sb = sa + G::kABytes;
          const int k0 = kb * kBlockK;
          if (!kPair) {
            ptx::mbar_arrive_expect_tx(local_bar, kTmaBytes);
            if (MODE == kNN) {
              if (!GATHER) ptx::tma_load_2d(sa, &map_a, local_bar, k0, t.row0);
#pragma unroll
              for (int j = 0; j < G::kBCols / 64; ++j)
                if (SWIGLU)
                  ptx::tma_load_3d(sb + j * kBoxBytes, j < 2 ? &map_b : &map_b2, local_bar,
                                   t.col0 / 2 + (j & 1) * 64, k0, t.expert);
                else
                  ptx::tma_load_3d(sb + j * kBoxBytes, &map_b, local_bar, t.col0 + j * 64, k0, t.expert);
            } else if (MODE == kNT) {
              if (!GATHER) ptx::tma_load_2d(sa, &map_a, local_bar, k0, t.row0);
              if (SWIGLU) {  // the maps' boxes are 128 rows of b high
                ptx::tma_load_3d(sb, &map_b, local_bar, k0, t.col0 / 2, t.expert);
                ptx::tma_load_3d(sb + G::kBBytes / 2, &map_b2, local_bar, k0, t.col0 / 2, t.expert);
              } else {
                ptx::tma_load_3d(sb, &map_b, local_bar, k0, t.col0, t.expert);
              }
            } else {
              const int r0 = t.k_row0 + k0;
              if (!GATHER) {
                if (p.wide_a) {
                  ptx::tma_load_3d(sa, tn_a, local_bar, 0, r0, t.row0 >> 6);
                } else {
#pragma unroll
                  for (int j = 0; j < kBlockM / 64; ++j)
                    ptx::tma_load_2d(sa + j * kBoxBytes, tn_a, local_bar, t.row0 + j * 64, r0);
                }
              }
              if (p.wide_b) {
                ptx::tma_load_3d(sb, tn_b, local_bar, 0, r0, t.col0 >> 6);
              } else {
#pragma unroll
                for (int j = 0; j < G::kBCols / 64; ++j)
                  ptx::tma_load_2d(sb + j * kBoxBytes, tn_b, local_bar, t.col0 + j * 64, r0);
              }
            }
          } else {
            // Pair: this CTA stages rows [row0+row_off, +128) of A and columns
            // [col0+col_off, +128) of B.
            // Both CTAs' loads complete on the leader's barrier (shared::cluster address).
            if (leader) ptx::mbar_arrive_expect_tx(local_bar, 2 * kTmaBytes);
            const uint32_t bar = ptx::mapa(local_bar, 0);
            if (MODE == kNN) {
              if (!GATHER) ptx::tma_load_2d_pair(sa, &map_a, bar, k0, t.row0 + row_off);
#pragma unroll
              for (int j = 0; j < G::kBCols / 64; ++j)
                if (SWIGLU)  // the leader stages the gate columns, its peer the up columns
                  ptx::tma_load_3d_pair(sb + j * kBoxBytes, leader ? &map_b : &map_b2, bar,
                                        t.col0 / 2 + j * 64, k0, t.expert);
                else
                  ptx::tma_load_3d_pair(sb + j * kBoxBytes, &map_b, bar, t.col0 + col_off + j * 64, k0,
                                        t.expert);
            } else if (MODE == kNT) {
              if (!GATHER) ptx::tma_load_2d_pair(sa, &map_a, bar, k0, t.row0 + row_off);
              if (SWIGLU) ptx::tma_load_3d_pair(sb, leader ? &map_b : &map_b2, bar, k0, t.col0 / 2, t.expert);
              else ptx::tma_load_3d_pair(sb, &map_b, bar, k0, t.col0 + col_off, t.expert);
            } else {
              const int r0 = t.k_row0 + k0;
              if (!GATHER) {
                if (p.wide_a) {
                  ptx::tma_load_3d_pair(sa, tn_a, bar, 0, r0, (t.row0 + row_off) >> 6);
                } else {
#pragma unroll
                  for (int j = 0; j < kBlockM / 64; ++j)
                    ptx::tma_load_2d_pair(sa + j * kBoxBytes, tn_a, bar, t.row0 + row_off + j * 64, r0);
                }
              }
              if (p.wide_b) {
                ptx::tma_load_3d_pair(sb, tn_b, bar, 0, r0, (t.col0 + col_off) >> 6);
              } else {
#pragma unroll
                for (int j = 0; j < G::kBCols / 64; ++j)
                  ptx::tma_load_2d_pair(sb + j * kBoxBytes, tn_b, bar, t.col0 + col_off + j * 64, r0);
              }
            }
          }
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
      feed.tally(warp);
    }
    __syncwarp();
  } else if (warp == 1 && leader) {
    // ---------------------------------------------------------- MMA issuer
    TileWalker walk(p, tail);
    TileFeed<kPair> feed(tail, wait, !leader);
    Tile t;
    uint32_t s = 0, ph = 0, it = 0;
    bool ok = true;
    // Tells the scheduler how many tiles have all their loads landed (it may then
    // edit the tensor-map copies those tiles loaded through).
    auto loads_landed = [&]() {
      if (MODE == kTN && lane == 0) *reinterpret_cast<volatile uint32_t*>(&tail->tiles_done) = feed.taken;
    };
    while (ok) {
      const int pos = feed.take(true, lane);
      if (pos == kNoTile) { ok = false; break; }
      if (!walk.decode(pos, &t)) break;
      const int nkb = tile_stages(t);
      if (nkb == 0) { loads_landed(); continue; }  // empty wgrad expert: the epilogue writes zeros
      const uint32_t ab = it & 1u, aph = (it >> 1) & 1u;
      ++it;
      const uint32_t te_bar = ptx::smem_u32(&tail->tmem_empty[ab]);
      // (acquire at cluster scope: half of the arrivals come from the other CTA's epilogue warps)
      if (!ptx::mbar_wait<kPair>(te_bar, aph ^ 1u, wait)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + ab * kBlockN;
      if (kLight && t.kind) {
        // D[128 output columns, rows rounded up to 16] = W[128, k] x X[rows, k]^T
        const int n_mma = (t.valid_rows + 15) & ~15;
        const uint32_t idesc = ptx::make_idesc_bf16(kLightCols, n_mma, MODE == kNN ? 1 : 0, 0);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&tail->full[s]), ph, wait)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t sw = stage_base + s * G::kStageBytes;
          const uint32_t sx = sw + kLightWBytes;
          if (lane == 0) {
#pragma unroll
            for (int k = 0; k < kLightK / 16; ++k) {
              const int h = k >> 2, j = k & 3;
              // NN: b[k, n] tile is MN-major (64-column boxes 8 KiB apart, +2048 B per
              // 16 of k); NT: b[n, k] tile is K-major (+32 B per 16 of k).
              const uint64_t adesc = (MODE == kNN)
                  ? ptx::make_smem_desc(sw + h * kLightWHalf, kBoxBytes, 1024u) + uint64_t(j) * (2048u >> 4)
                  : ptx::make_smem_desc(sw + h * kLightWHalf, 16u, 1024u) + uint64_t(j) * (32u >> 4);
              const uint64_t bdesc = ptx::make_smem_desc(sx + h * kLightXHalf, 16u, 1024u) + uint64_t(j) * (32u >> 4);
              ptx::mma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            ptx::mma_commit(ptx::smem_u32(&tail->empty[s]));
          }
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (ok && lane == 0) ptx::mma_commit(ptx::smem_u32(&tail->tmem_full[ab]));
        __syncwarp();
        continue;
      }
      for (int kb = 0; kb < nkb; ++kb) {
        const uint32_t f_bar = ptx::smem_u32(&tail->full[s]);
        // (gather variant of a pair: one arrival is the other CTA's gather warp)
        if (!ptx::mbar_wait<kPair && GATHER>(f_bar, ph, wait)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t sa = stage_base + s * G::kStageBytes;
        const uint32_t sb = sa + G::kABytes;
        if (lane == 0) {
          // K-major SW128 operand: 8-row groups 1024 B apart, +32 B per 16-wide k step.
          // MN-major SW128 operand: 64-wide boxes 8 KiB apart (LBO), 8-k-row groups
          // 1024 B apart (SBO), +2048 B per 16-deep k step.
          const uint64_t adesc = kAMn ? ptx::make_smem_desc(sa, kBoxBytes, 1024u)
                                      : ptx::make_smem_desc(sa, 16u, 1024u);
          const uint64_t bdesc = kBMn ? ptx::make_smem_desc(sb, kBoxBytes, 1024u)
                                      : ptx::make_smem_desc(sb, 16u, 1024u);
          constexpr uint64_t a_step = kAMn ? (2048u >> 4) : (32u >> 4);
          constexpr uint64_t b_step = kBMn ? (2048u >> 4) : (32u >> 4);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            if (kPair)
              ptx::mma_bf16_ss_pair(d_tmem, adesc + k * a_step, bdesc + k * b_step, kIdesc,
                                    (kb | k) != 0 ? 1u : 0u);
            else
              ptx::mma_bf16_ss(d_tmem, adesc + k * a_step, bdesc + k * b_step, kIdesc,
                               (kb | k) != 0 ? 1u : 0u);
          }
          if (kPair) ptx::mma_commit_pair(ptx::smem_u32(&tail->empty[s]), 0x3);
          else ptx::mma_commit(ptx::smem_u32(&tail->empty[s]));
        }
        __syncwarp();
        if (++s == kStages) { s = 0; ph ^= 1u; }
      }
      if (ok) loads_landed();
      if (ok && lane == 0) {
        if (kPair) ptx::mma_commit_pair(ptx::smem_u32(&tail->tmem_full[ab]), 0x3);
        else ptx::mma_commit(ptx::smem_u32(&tail->tmem_full[ab]));
      }
      __syncwarp();
    }
    if (lane == 0) feed.tally(warp);
  } else if (warp == 1) {
    // peer CTA of a pair: the leader issues the MMAs for both
  } else if (warp == kSchedWarp) {
    // ---------------------------------------------------------- scheduler
    if (leader) {
      if (MODE == kTN) {
        // Copies of both maps in every slot (2 KiB per cluster), by the whole warp.
        const uint4* src_a = reinterpret_cast<const uint4*>(&map_a);
        const uint4* src_b = reinterpret_cast<const uint4*>(&map_b);
        uint4* dst = reinterpret_cast<uint4*>(my_maps);
        for (int i = lane; i < kMapSlots * 2 * 8; i += 32) {
          const int which = (i >> 3) & 1;  // 8 x 16 bytes per map; maps alternate a, b
          dst[i] = which ? src_b[i & 7] : src_a[i & 7];
        }
        __syncwarp();
      }
      if (lane == 0) {
        TileWalker walk(p, tail);
        TileFeed<kPair> feed(tail, wait, !leader);
        Tile t;
        // wgrad: the map slot clipped to the current expert, and for every slot the
        // index (in this cluster's sequence of tiles) of the last tile that loads
        // through it.
        int held_expert = -1;
        int held_slot = 0;
        int last_tile[kMapSlots];
#pragma unroll
        for (int i = 0; i < kMapSlots; ++i) last_tile[i] = -1;
        int pos = first_tile;
        // Positions after the first come from the global counter, drawn one tile
        // ahead of their use so that the atomic's round trip is never waited for.
        uint32_t drawn = (pos < walk.total) ? atomicAdd(sched_counter, 1u) : 0u;
        bool ok = true;
        while (ok) {
          int entry = 0;
          const bool live = walk.decode(pos, &t);
          if (MODE == kTN && live && t.k_len > 0) {
            if (held_expert != t.expert) {
              // New expert: clip the row extent of a and b at its last row, in the next
              // copy of the maps.  That copy may only be edited once every tile that
              // loaded through it has all its loads landed; with kMapSlots copies this
              // is a wait only when the MMA warp is that many experts behind (the tiles
              // in question have been handed out already and finish on their own).
              const int slot = (held_slot + 1) % kMapSlots;
              const uint64_t t0 = ptx::globaltimer_ns();
              while (last_tile[slot] >= static_cast<int>(*reinterpret_cast<volatile uint32_t*>(&tail->tiles_done))) {
                if (tail->abort_flag || ptx::globaltimer_ns() - t0 > wait.limit_ns) {
                  tail->abort_flag = 1u;
                  ok = false;
                  break;
                }
                __nanosleep(64);
              }
              if (!ok) break;
              held_expert = t.expert;
              held_slot = slot;
              CUtensorMap* ea = my_maps + slot * 2;
              CUtensorMap* eb = ea + 1;
              const uint32_t rows_end = static_cast<uint32_t>(t.k_row0 + t.k_len);
              ptx::tensormap_set_dim1(ea, rows_end);
              ptx::tensormap_set_dim1(eb, rows_end);
              ptx::fence_tensormap_release();
              entry = kMapFresh;
            }
            entry |= held_slot;
            last_tile[held_slot] = static_cast<int>(feed.taken);
          }
          if (!feed.publish(pos, entry)) { ok = false; break; }
          if (!live) break;  // the end of the order has been handed to everyone
          pos = static_cast<int>(drawn) + tile_stride;
          if (pos < walk.total) drawn = atomicAdd(sched_counter, 1u);
        }
      }
      __syncwarp();
    }
  } else if (PUSH && warp > kSchedWarp) {
    // ---------------------------------------------------------- row push
    // Two forms.  Default: one thread per thread block issues bulk async copies
    // (below).  Otherwise the four push warps copy through registers: items are
    // dealt warp by warp over the whole grid, a lane issues all of its loads of a
    // sweep (kPushVecsInFlight x 16 bytes) before the first store, and the stores are
    // not waited for.  Either way the rows are complete when the kernel is: the
    // caller's barrier after it publishes them.  interval_ns > 0 paces the items
    // over time (measured: no better than sending as fast as it goes).
    if (push.via_tma) {
      // Bulk-copy form: one thread moves this thread block's share of the items in
      // chunks of 2 KiB, global -> shared (completing on an mbarrier) -> peer, three
      // chunks in flight; no register staging and nothing through the load/store path.
      if (warp == kSchedWarp + 1 && lane == 0) {
        const uint32_t stage = ptx::smem_u32(reinterpret_cast<uint8_t*>(tail) + kPushStageOffset);
        const int64_t row_bytes = push.row_vecs * 16;
        const int64_t chunks_per_row = (row_bytes + kPushChunkBytes - 1) / kPushChunkBytes;
        const int64_t my_items = (push.n_items > blockIdx.x) ? (push.n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const int64_t total = my_items * chunks_per_row;
        const uint64_t t0 = ptx::globaltimer_ns();
        // chunk q of this block's sequence: item blockIdx.x + (q / chunks_per_row) * gridDim.x, piece q % chunks_per_row
        auto issue_load = [&](int64_t q) {
          const int64_t it = q / chunks_per_row, piece = q - it * chunks_per_row;
          if (piece == 0 && push.interval_ns > 0) {
            const uint64_t due = t0 + static_cast<uint64_t>(it) * static_cast<uint64_t>(push.interval_ns) / kPushWarps;  // this thread has four warps' shares
            while (ptx::globaltimer_ns() < due) __nanosleep(500);   // bounded: the pacing as a whole stays inside the wait limit
          }
          const int64_t item = blockIdx.x + it * int64_t(gridDim.x);
          const int64_t sr = (push.src_row != nullptr) ? push.src_row[item] : item;
          const int64_t off = piece * kPushChunkBytes;
          const uint32_t bytes = static_cast<uint32_t>(row_bytes - off < kPushChunkBytes ? row_bytes - off : kPushChunkBytes);
          const int b = static_cast<int>(q % kPushChunks);
          const uint32_t bar = ptx::smem_u32(&tail->push_full[b]);
          ptx::mbar_arrive_expect_tx(bar, bytes);
          ptx::bulk_load_1d(stage + b * kPushChunkBytes, reinterpret_cast<const uint8_t*>(push.src + sr * push.row_vecs) + off,
                            bytes, bar);
        };
        bool ok = true;
        // loads run two chunks ahead of the stores
        for (int64_t q = 0; q < total && q < kPushChunks - 1; ++q) issue_load(q);
        for (int64_t q = 0; q < total && ok; ++q) {
          if (q + kPushChunks - 1 < total) {
            // the buffer chunk q + 2 will land in was last read by the store of chunk q - 1
            if (q >= 1) ptx::bulk_wait_group_read<0>();
            issue_load(q + kPushChunks - 1);
          }
          const int b = static_cast<int>(q % kPushChunks);
          const uint32_t ph = static_cast<uint32_t>((q / kPushChunks) & 1);
          if (!ptx::mbar_wait(ptx::smem_u32(&tail->push_full[b]), ph, wait)) { ok = false; break; }
          const int64_t it = q / chunks_per_row, piece = q - it * chunks_per_row;
          const int64_t item = blockIdx.x + it * int64_t(gridDim.x);
          const int64_t off = piece * kPushChunkBytes;
          const uint32_t bytes = static_cast<uint32_t>(row_bytes - off < kPushChunkBytes ? row_bytes - off : kPushChunkBytes);
          uint8_t* dst = static_cast<uint8_t*>(push.peer_base[push.dst_rank[item]]) + push.dst_row[item] * row_bytes + off;
          ptx::bulk_store_1d(dst, stage + b * kPushChunkBytes, bytes);
          ptx::bulk_commit_group();
        }
        ptx::bulk_wait_group_all();
      }
    } else {
    const int64_t first = int64_t(blockIdx.x) * kPushWarps + (warp - (kSchedWarp + 1));
    const int64_t step = int64_t(gridDim.x) * kPushWarps;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint64_t due = t0;
    for (int64_t item = first; item < push.n_items; item += step) {
      if (push.interval_ns > 0) {
        // bounded: `due` lies at most (items per warp) x interval past t0
        while (ptx::globaltimer_ns() < due) __nanosleep(500);
        due += static_cast<uint64_t>(push.interval_ns);
      }
      const int64_t sr = (push.src_row != nullptr) ? push.src_row[item] : item;
      const uint4* src = push.src + sr * push.row_vecs;
      uint4* dst = static_cast<uint4*>(push.peer_base[push.dst_rank[item]]) + push.dst_row[item] * push.row_vecs;
      for (int64_t base = 0; base < push.row_vecs; base += int64_t(kPushVecsInFlight) * 32) {
        uint4 r[kPushVecsInFlight];
#pragma unroll
        for (int j = 0; j < kPushVecsInFlight; ++j) {
          const int64_t v = base + j * 32 + lane;
          if (v < push.row_vecs) r[j] = __ldg(src + v);
        }
#pragma unroll
        for (int j = 0; j < kPushVecsInFlight; ++j) {
          const int64_t v = base + j * 32 + lane;
          if (v < push.row_vecs) dst[v] = r[j];
        }
      }
    }
    }
  } else if (GATHER && warp > kSchedWarp) {
    // ---------------------------------------------------------- A-row gather
    // The caller's sort-by-expert fused into the load: row i of the grouped
    // operand is row a_rows[i] of a_src (rows of p.d1 elements).  Gather warp w
    // owns ring stage w: it fills it for every k-block that lands there (every
    // kStages-th of the stream of k-blocks, which runs on across tiles), waits for
    // its own copies and reports the stage full, so that as with the TMA loads
    // every stage can be in flight at once.  A warp copies this CTA's 128 x 64
    // tile with 16-byte cp.async: eight neighbouring lanes cover the 128 bytes of
    // one row, a lane serves rows sub, sub + 4, .. sub + 124, and writes the
    // K-major 128-byte-swizzled layout a TMA box load would leave (16-byte chunk
    // index ^= row % 8).
    const int w = warp - (kSchedWarp + 1);  // the stage this warp owns
    const int chunk = lane & 7;
    const int sub = lane >> 3;
    const uint32_t stage_addr = stage_base + uint32_t(w) * G::kStageBytes;
    const uint32_t full_bar = kPair ? ptx::mapa(ptx::smem_u32(&tail->full[w]), 0) : ptx::smem_u32(&tail->full[w]);
    const uint32_t empty_bar = ptx::smem_u32(&tail->empty[w]);
    TileWalker walk(p, tail);
    TileFeed<kPair> feed(tail, wait, !leader);
    Tile t;
    uint32_t ph = 0;  // parity of this stage's current use
    int next = w;     // position in the stream of k-blocks of this warp's next one
    int base = 0;     // k-blocks of the stream before the current tile
    bool ok = true;
    bool bad_index = false;
    while (ok) {
      const int pos = feed.take(true, lane);
      if (pos == kNoTile) { ok = false; break; }
      if (!walk.decode(pos, &t)) break;
      const int nkb = tile_stages(t);
      if (MODE == kTN) {
        // wgrad: the gathered rows are the contraction.  A k-block is 64 grouped rows
        // (k_row0 + 64 kb ..) by this CTA's 128 columns of a_src, staged as two
        // MN-major boxes of 64 columns: row r of box j at j * 8 KiB + 128 r, chunk
        // index ^= r % 8.  A lane serves rows sub, sub + 4, .. sub + 60 of both boxes.
        // Rows past the expert's last one are zeros (what the clipped tensor map
        // does for the operand that TMA loads).
        int idx[16];  // source rows of this lane's 16 rows of the k-block, -1 = zeros
        auto load_idx = [&](int kb) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int r = kb * kBlockK + i * 4 + sub;  // row inside the expert
            idx[i] = -1;
            if (r < t.k_len) {
              const int ix = a_rows[t.k_row0 + r];
              if (ix >= 0 && ix < a_src_rows) idx[i] = ix;
              else bad_index = true;
            }
          }
        };
        if (next < base + nkb) load_idx(next - base);
        for (; next < base + nkb; next += kStages) {
          if (lane == 0) ok = ptx::mbar_wait(empty_bar, ph ^ 1u, wait);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
#pragma unroll
          for (int j = 0; j < kBlockM / 64; ++j) {
            const int col = t.row0 + row_off + j * 64 + chunk * 8;  // column of a_src
            const bool in_m = col < p.d1;  // d1 is a multiple of 8
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int r = i * 4 + sub;
              const uint32_t dst = stage_addr + uint32_t(j) * kBoxBytes + uint32_t(r) * 128u +
                                   (uint32_t(chunk ^ (r & 7)) << 4);
              const bool live = in_m && idx[i] >= 0;
              ptx::cp_async_16(dst, live ? static_cast<const void*>(a_src + int64_t(idx[i]) * p.d1 + col) : a_src,
                               live ? 16u : 0u);
            }
          }
          // the indices of this warp's next k-block of the tile arrive while the copies fly
          if (next + kStages < base + nkb) load_idx(next + kStages - base);
          ptx::cp_async_wait_all();
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (kPair) ptx::mbar_arrive_cluster(full_bar);
            else ptx::mbar_arrive(full_bar);
          }
          ph ^= 1u;
        }
        base += nkb;
        continue;
      }
      if (next < base + nkb) {
        int idx[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int r = row_off + j * 4 + sub;  // row inside the (pair) tile
          // rows that do not exist are filled with zeros and never stored; so is a
          // row whose index lies outside a_src, which is also reported
          idx[j] = -1;
          if (r < t.valid_rows) {
            const int ix = a_rows[t.row0 + r];
            if (ix >= 0 && ix < a_src_rows) idx[j] = ix;
            else bad_index = true;
          }
        }
        for (; next < base + nkb; next += kStages) {
          if (lane == 0) ok = ptx::mbar_wait(empty_bar, ph ^ 1u, wait);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
          const int kcol = (next - base) * kBlockK + chunk * 8;
          const bool in_k = kcol < p.d1;  // d1 is a multiple of 8: a chunk is all in or all out
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int r = j * 4 + sub;
            const uint32_t dst = stage_addr + uint32_t(r) * 128u + (uint32_t(chunk ^ (r & 7)) << 4);
            const bool live = in_k && idx[j] >= 0;
            ptx::cp_async_16(dst, live ? static_cast<const void*>(a_src + int64_t(idx[j]) * p.d1 + kcol) : a_src,
                             live ? 16u : 0u);
          }
          ptx::cp_async_wait_all();
          // this lane's copies are complete: make them visible to the tensor core's
          // proxy, then one arrival for the warp on the (leader's) full barrier
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (kPair) ptx::mbar_arrive_cluster(full_bar);
            else ptx::mbar_arrive(full_bar);
          }
          ph ^= 1u;
        }
      }
      base += nkb;
    }
    ptx::cp_async_wait_all();
    if (bad_index && status != nullptr) atomicOr(status, 0x8u);
  } else {
    // ---------------------------------------------------------- epilogue
    const int q = warp & 3;            // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which 128 of the tile's 256 columns
    const int col_base = half * (kBlockN / 2);
    const uint32_t my_out = out_base + uint32_t(warp - 2) * (G::kOutBufBytes * G::kOutBufs);
    TileWalker walk(p, tail);
    TileFeed<kPair> feed(tail, wait, !leader);
    Tile t;
    uint32_t it = 0;
    uint32_t stores = 0;  // TMA stores this warp has issued (lane 0's bulk groups)
    bool ok = true;
    bool bad_dest = false;  // a row_dest entry outside the window the caller declared
    // A scattered row may only go to a 16-byte aligned address (the bulk copies that
    // carry it need that) inside [dest_lo, dest_hi) (dest_hi == 0: the caller vouches
    // for the range of its table, e.g. rows in a peer GPU's buffer).
    const int64_t dest_row_bytes = (SWIGLU ? (p.n >> 1) : p.n) * 2;
    auto dest_ok = [&](int64_t addr) {
      return (addr & 15) == 0 && (dest_hi == 0 || (addr >= dest_lo && addr + dest_row_bytes <= dest_hi));
    };
    // Buffer for the next TMA store and the wait before it may be written: with two
    // buffers the store before last read this one.
    auto stage_buf = [&]() { return my_out + (G::kOutBufs == 2 ? (stores & 1u) * G::kOutBufBytes : 0u); };

    // One 32-column chunk `v` (fp32 bits) of this lane's row, starting at column
    // `col` of the tile: through the staging buffer and a TMA store when the
    // whole warp's rows exist, else straight to global for the rows that do.
    const bool scatter_rows = (MODE != kTN) && (row_dest != nullptr);
    // 32 fp32 values -> 32 bf16 in four 16-byte pieces
    auto pack = [](const uint32_t (&v)[32], uint4* o) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h;
        h = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 0]), __uint_as_float(v[j * 8 + 1]));
        o[j].x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 2]), __uint_as_float(v[j * 8 + 3]));
        o[j].y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 4]), __uint_as_float(v[j * 8 + 5]));
        o[j].z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 6]), __uint_as_float(v[j * 8 + 7]));
        o[j].w = *reinterpret_cast<uint32_t*>(&h);
      }
    };
    // wgrad, all 32 rows of the warp exist: 64 columns (two chunks) through one
    // staging buffer of 128-byte rows (128-byte swizzle: 16-byte piece index ^=
    // row % 8) and one TMA store of a 64 x 32 box; columns past the tensor's last
    // are clipped by the store.
    auto emit64 = [&](const uint32_t (&v0)[32], const uint32_t (&v1)[32], int col, int tile_row, int col0) {
      uint4 o[8];
      pack(v0, o);
      pack(v1, o + 4);
      const uint32_t buf = stage_buf();
      if (lane == 0 && stores > 0) ptx::bulk_wait_group_read<G::kOutBufs - 1>();
      __syncwarp();
      const uint32_t row_addr = buf + uint32_t(lane) * 128u;
      const uint32_t sw = uint32_t(lane) & 7u;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t dst = row_addr + ((uint32_t(j) ^ sw) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[j].x), "r"(o[j].y),
                     "r"(o[j].z), "r"(o[j].w)
                     : "memory");
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        ptx::tma_store_2d(&map_c, buf, col0 + col, tile_row);
        ptx::bulk_commit_group();
      }
      ++stores;
    };
    auto emit = [&](const uint32_t (&v)[32], int col, bool warp_full, bool row_ok,
                    __nv_bfloat16* crow, int cols_left, int tile_row, int col0) {
      if (col >= cols_left) return;  // chunk lies entirely past the last column
      uint4 o[4];
      pack(v, o);
      if (MODE != kTN && warp_full) {
        // The store that last read this buffer must be done reading.
        const uint32_t buf = stage_buf();
        if (lane == 0 && stores > 0) ptx::bulk_wait_group_read<G::kOutBufs - 1>();
        __syncwarp();
        // 64-byte swizzle: 16-byte chunk index ^= (row / 2) % 4.
        const uint32_t row_addr = buf + uint32_t(lane) * 64u;
        const uint32_t sw = (uint32_t(lane) >> 1) & 3u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t dst = row_addr + ((uint32_t(j) ^ sw) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[j].x), "r"(o[j].y),
                       "r"(o[j].z), "r"(o[j].w)
                       : "memory");
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(&map_c, buf, col0 + col, tile_row);
          ptx::bulk_commit_group();
        }
        ++stores;
      } else if (scatter_rows) {
        // Row-scatter mode: this lane's 64-byte piece goes through its own slice
        // of the staging buffer (linear, no swizzle) and leaves as one bulk
        // async copy, so the thread never waits on the (possibly remote) write.
        if (row_ok) {
          if (stores > 0) ptx::bulk_wait_group_read<0>();  // this lane's previous copy
          const uint32_t row_addr = my_out + uint32_t(lane) * 64u;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t(j) << 4)),
                         "r"(o[j].x), "r"(o[j].y), "r"(o[j].z), "r"(o[j].w)
                         : "memory");
          ptx::fence_proxy_async_smem();
          const int left = cols_left - col;
          const uint32_t bytes = left < 32 ? uint32_t(left) * 2u : 64u;
          if (reduce_add) ptx::bulk_reduce_add_bf16_1d(crow + col, row_addr, bytes);
          else ptx::bulk_store_1d(crow + col, row_addr, bytes);
          ptx::bulk_commit_group();
        }
        ++stores;
      } else if (row_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int cj = col + j * 8;
          if (cj < cols_left) *reinterpret_cast<uint4*>(crow + cj) = o[j];
        }
      }
    };

    while (ok) {
      const int pos = feed.take(true, lane);
      if (pos == kNoTile) { ok = false; break; }
      if (!walk.decode(pos, &t)) break;
      const int nkb = tile_stages(t);
      if (kLight && t.kind) {
        // Transposed tile: TMEM lane = output column, TMEM column = output row.  This
        // warp reads the 32 output columns of its lane quadrant for its half of the
        // rows, eight rows at a time, and every lane writes its column of each row:
        // a warp's store covers 64 consecutive bytes of one output row.  (The rows
        // of all such tiles together are a sliver of the output.)
        const uint32_t ab = it & 1u, aph = (it >> 1) & 1u;
        ++it;
        if (!ptx::mbar_wait<false, 64>(ptx::smem_u32(&tail->tmem_full[ab]), aph, wait)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const int n_mma = (t.valid_rows + 15) & ~15;
        const int half_rows = n_mma >> 1;  // a multiple of 8
        const int r_base = half * half_rows;
        const int col = t.col0 + q * 32 + lane;
        const bool col_ok = col < p.n;
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + ab * kBlockN + uint32_t(r_base);
        for (int i = 0; i < half_rows; i += 8) {
          uint32_t v[8];
          ptx::tmem_ld_32x8(taddr + uint32_t(i), v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int r = r_base + i + u;
            if (r < t.valid_rows && col_ok) {
              const int64_t grow = int64_t(t.row0) + r;
              float f = __uint_as_float(v[u]);
              __nv_bfloat16* dst;
              if (row_dest != nullptr) {
                const int64_t addr = row_dest[grow];
                if (!dest_ok(addr)) { bad_dest = true; continue; }
                if (row_scale != nullptr) f *= row_scale[grow];
                dst = reinterpret_cast<__nv_bfloat16*>(addr) + col;
              } else {
                dst = c + grow * p.n + col;
              }
              const __nv_bfloat16 h = __float2bfloat16_rn(f);
              if (row_dest != nullptr && reduce_add) atomicAdd(dst, h);
              else *dst = h;
            }
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tail->tmem_empty[ab]));
        continue;
      }
      const int r = row_off + q * 32 + lane;  // row inside the (pair) tile
      bool row_ok = r < t.valid_rows;
      // row_dest != nullptr (expert-parallel combine fused into this epilogue):
      // output row i does not go to c[i] but to the address row_dest[i], which may
      // be a row of a buffer on another GPU; such rows are written with plain
      // stores by the lane that holds them.
      const bool scatter = (MODE != kTN) && (row_dest != nullptr);
      const bool warp_full = !scatter && (row_off + q * 32 + 31) < t.valid_rows;
      const int64_t out_row0 = (MODE == kTN) ? (int64_t(t.expert) * p.d1 + t.row0) : int64_t(t.row0);
      // Output geometry: the gated product writes half as many columns as it schedules.
      const int64_t out_n = SWIGLU ? (p.n >> 1) : p.n;
      const int out_col0 = SWIGLU ? (t.col0 >> 1) : t.col0;
      __nv_bfloat16* crow = c + (out_row0 + r) * out_n + out_col0;
      if (scatter && row_ok) {
        const int64_t addr = row_dest[out_row0 + r];
        if (dest_ok(addr)) {
          crow = reinterpret_cast<__nv_bfloat16*>(addr) + out_col0;
        } else {  // never written: skipped and reported
          row_ok = false;
          bad_dest = true;
        }
      }
      const int tile_row = static_cast<int>(out_row0) + row_off + q * 32;  // first row of this warp
      const int cols_left = static_cast<int>(out_n) - out_col0;  // multiple of 8
      // Scatter mode with per-row weights (the router's top-k weight of this row).
      const bool scaled = scatter && row_scale != nullptr;
      const float row_w = (scaled && row_ok) ? row_scale[out_row0 + r] : 1.0f;
      auto scale = [&](uint32_t (&v)[32]) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * row_w);
      };
      uint32_t va[32], vb[32];
      if (MODE == kTN && nkb == 0) {  // (forward and dgrad tiles always have k > 0)
        // Empty wgrad expert: its block of the output is zeros.
        if (warp_full) {
          // Zeros need staging once: every store of this tile reads the same buffer,
          // so none of them waits for the one before.
          const uint32_t buf = stage_buf();
          if (lane == 0 && stores > 0) ptx::bulk_wait_group_read<G::kOutBufs - 1>();
          __syncwarp();
          const uint32_t row_addr = buf + uint32_t(lane) * 128u;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(row_addr + (uint32_t(j) << 4)), "r"(0u)
                         : "memory");
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
#pragma unroll 1
            for (int ch = 0; ch < kBlockN / 128; ++ch) {
              const int col = col_base + ch * 64;
              if (col < cols_left) ptx::tma_store_2d(&map_c, buf, t.col0 + col, tile_row);
            }
            ptx::bulk_commit_group();
          }
          ++stores;
          continue;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) va[i] = 0u;
#pragma unroll 1
        for (int ch = 0; ch < kBlockN / 64; ++ch)
          emit(va, col_base + ch * 32, warp_full, row_ok, crow, cols_left, tile_row, t.col0);
        continue;
      }
      const uint32_t ab = it & 1u, aph = (it >> 1) & 1u;
      ++it;
      if (!ptx::mbar_wait<false, 64>(ptx::smem_u32(&tail->tmem_full[ab]), aph, wait)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      if (SWIGLU) {
        // This warp's 64 of the tile's 128 output columns: gate from accumulator
        // columns [64 half, +64), up from the same columns of the second half.
        const uint32_t tg = tmem_base + (uint32_t(q * 32) << 16) + ab * kBlockN + half * 64;
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
          ptx::tmem_ld_32x32(tg + ch * 32, va);
          ptx::tmem_ld_32x32(tg + kBlockN / 2 + ch * 32, vb);
          ptx::tmem_ld_wait();
          if (ch == 1) {
            // Every column has been read: hand the accumulator back before the last stores.
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              const uint32_t te_bar = ptx::smem_u32(&tail->tmem_empty[ab]);
              if (kPair) ptx::mbar_arrive_cluster(ptx::mapa(te_bar, 0));
              else ptx::mbar_arrive(te_bar);
            }
          }
          const int col = half * 64 + ch * 32;
          if (gate_grad != nullptr) {
            // Backward of the gated product: with g, u recomputed in the accumulator and
            // dh = gate_grad[row, col ..] read here, the gradients w.r.t. the two products
            //   dg = dh * u * silu'(g),  silu'(g) = s (1 + g (1 - s)),  s = 1 / (1 + exp(-g))
            //   du = dh * silu(g)
            // go to rows [0, T) and [T, 2T) of the output.
            uint4 d4[4] = {};
            if (row_ok) {
              const uint4* src = reinterpret_cast<const uint4*>(gate_grad + (out_row0 + r) * out_n + out_col0 + col);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (col + j * 8 < cols_left) d4[j] = src[j];
            }
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(d4);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float g = __uint_as_float(va[i]);
              const float u = __uint_as_float(vb[i]);
              const float2 dpair = __bfloat1622float2(d2[i >> 1]);
              const float dh = (i & 1) ? dpair.y : dpair.x;
              const float sg = __fdividef(1.0f, 1.0f + __expf(-g));
              va[i] = __float_as_uint(dh * u * sg * (1.0f + g * (1.0f - sg)));
              vb[i] = __float_as_uint(dh * g * sg);
            }
            emit(va, col, warp_full, row_ok, crow, cols_left, tile_row, out_col0);
            emit(vb, col, warp_full, row_ok, crow + p.tokens * out_n, cols_left, tile_row + static_cast<int>(p.tokens),
                 out_col0);
            continue;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float g = __uint_as_float(va[i]);
            const float u = __uint_as_float(vb[i]);
            va[i] = __float_as_uint(__fdividef(g, 1.0f + __expf(-g)) * u);  // silu(g) * u
          }
          if (scaled) scale(va);
          emit(va, col, warp_full, row_ok, crow, cols_left, tile_row, out_col0);
        }
        continue;
      }
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + ab * kBlockN + col_base;
      if (MODE == kTN && warp_full) {
#pragma unroll 1
        for (int ch = 0; ch < kBlockN / 64; ch += 2) {
          ptx::tmem_ld_32x32(taddr + ch * 32, va);
          ptx::tmem_ld_32x32(taddr + (ch + 1) * 32, vb);
          ptx::tmem_ld_wait();
          if (ch + 2 >= kBlockN / 64) {
            // Every column has been read: hand the accumulator back before the last store.
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              const uint32_t te_bar = ptx::smem_u32(&tail->tmem_empty[ab]);
              if (kPair) ptx::mbar_arrive_cluster(ptx::mapa(te_bar, 0));
              else ptx::mbar_arrive(te_bar);
            }
          }
          if (col_base + ch * 32 < cols_left) emit64(va, vb, col_base + ch * 32, tile_row, t.col0);
        }
        continue;
      }
      ptx::tmem_ld_32x32(taddr, va);
#pragma unroll 1
      for (int ch = 0; ch < kBlockN / 64; ch += 2) {
        ptx::tmem_ld_wait();
        ptx::tmem_ld_32x32(taddr + (ch + 1) * 32, vb);
        if (scaled) scale(va);
        emit(va, col_base + ch * 32, warp_full, row_ok, crow, cols_left, tile_row, t.col0);
        ptx::tmem_ld_wait();
        if (ch + 2 < kBlockN / 64) {
          ptx::tmem_ld_32x32(taddr + (ch + 2) * 32, va);
        } else {
          // Every column has been read: hand the accumulator back before the last stores.
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            const uint32_t te_bar = ptx::smem_u32(&tail->tmem_empty[ab]);
            if (kPair) ptx::mbar_arrive_cluster(ptx::mapa(te_bar, 0));
            else ptx::mbar_arrive(te_bar);
          }
        }
        if (scaled) scale(vb);
        emit(vb, col_base + (ch + 1) * 32, warp_full, row_ok, crow, cols_left, tile_row, t.col0);
      }
    }
    // Shared memory must outlive the stores that still read it.
    if (lane == 0 || scatter_rows) ptx::bulk_wait_group_all();
    if (bad_dest && status != nullptr) atomicOr(status, 0x10u);
    if (lane == 0) feed.tally(warp);
    __syncwarp();
  }

  // ------------------------------------------------------------ teardown
  __syncthreads();
  if (threadIdx.x == 0 && status != nullptr) {
    // Self-check: the producer, the MMA issuer and the eight epilogue warps of a
    // CTA were handed the same positions (same count, same sum), in order.
    bool fault = tail->handoff_fault != 0u;
    if (!tail->abort_flag) {
      const uint32_t ref = tail->role_sum[0];
      for (int wq = leader ? 1 : 2; wq < 2 + kEpilogueWarps; ++wq) fault = fault || (tail->role_sum[wq] != ref);
    }
    if (fault) atomicOr(status, 0x20u);
  }
  if (tail->abort_flag) {
    // A wait gave up.  Report it, then give copies and MMAs still in flight time
    // to land before shared memory and TMEM are handed back.
    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, 0x1u);
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  // Neither CTA of a pair may retire while the other can still signal its
  // barriers or read its shared memory.
  if (kPair) ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if (kPair) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    else ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Argument fill on its own (bit-exact tests, inspection): the same scan step the
// GEMM kernels' schedule is built from, writing the reference's nine per-expert
// values (schedule.cuh: fill_fields).
__global__ void __launch_bounds__(32, 1)
fill_offsets_kernel(const int64_t* __restrict__ batch_sizes, const Problem p, int64_t* __restrict__ out) {
  const int lane = threadIdx.x;
  int64_t carry = 0;
  for (int base = 0; base < p.z; base += 32) {
    const int e = base + lane;
    const int64_t v = (e < p.z) ? batch_sizes[e] : 0;
    const int64_t start = scan_step(v, lane, &carry);
    if (e < p.z) fill_fields(p, e, start, v, out + int64_t(e) * 9);
  }
}

// The schedule a GEMM launch with this Problem walks, written out for tests: runs
// the kernels' own build_schedule and TileWalker in one CTA and stores, for every
// position of the launch order, {expert, row0, col0, valid_rows, stages, kind}.
// out_count receives the number of tiles; at most max_tiles are written.
__global__ void __launch_bounds__(kThreads, 1)
schedule_dump_kernel(const int64_t* __restrict__ batch_sizes, const Problem p, int32_t* __restrict__ out,
                     int max_tiles, int32_t* __restrict__ out_count, uint32_t* status) {
  __shared__ SmemTail tail;
  build_schedule(p, batch_sizes, &tail, status);
  __syncthreads();
  if (threadIdx.x == 0) {
    TileWalker walk(p, &tail);
    Tile t;
    int n = 0;
    for (int pos = 0; walk.decode(pos, &t); ++pos) {
      if (n < max_tiles) {
        int32_t* o = out + int64_t(n) * 6;
        o[0] = t.expert; o[1] = t.row0; o[2] = t.col0; o[3] = t.valid_rows; o[4] = tile_stages(t); o[5] = t.kind;
      }
      ++n;
    }
    *out_count = n;
  }
}

// A wait that nothing ends, with the caller's limit: one warp waits on an mbarrier
// nobody arrives on, gives up after limit_ns and reports STATUS_TIMEOUT exactly as
// the GEMM kernels' roles do.  Nothing is in flight, so the launch ends cleanly.
__global__ void __launch_bounds__(32, 1) wait_timeout_kernel(uint64_t limit_ns, uint32_t* status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    abort_flag = 0u;
    ptx::fence_mbar_init();
  }
  __syncwarp();
  const ptx::WaitCtx wait{&abort_flag, limit_ns};
  const bool ok = ptx::mbar_wait(ptx::smem_u32(&bar), 0u, wait);
  __syncwarp();
  if (threadIdx.x == 0 && (!ok || abort_flag) && status != nullptr) atomicOr(status, 0x1u);
}

}  // namespace b200gmm
