// C-ABI entry points of libb200gmm (declared in include/b200gmm.h): argument
// checks, TMA tensor-map construction and kernel launches.  No torch types, no
// exceptions, no allocation: scratch comes from the caller.
#include "../../include/b200gmm.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <mutex>
#include <vector>

#include "ep_exchange.cuh"
#include "gmm_kernel.cuh"

namespace {

using namespace b200gmm;

std::atomic<int64_t> g_launches{0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

typedef CUresult (*CtxGetCurrentFn)(CUcontext*);

CtxGetCurrentFn ctx_get_current_fn() {
  static CtxGetCurrentFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<CtxGetCurrentFn>(p);
  }();
  return fn;
}

// cuTensorMapEncodeTiled is a driver call and fails with "invalid context" on a
// thread that has a CUDA device selected but no context bound yet (e.g. an
// autograd worker whose allocations all came from a cache).  Binding the
// device's primary context to the calling thread is what cudaSetDevice does.
int ensure_context(int dev) {
  CtxGetCurrentFn get = ctx_get_current_fn();
  CUcontext ctx = nullptr;
  if (get != nullptr && get(&ctx) == CUDA_SUCCESS && ctx != nullptr) return B200GMM_OK;
  if (cudaSetDevice(dev) != cudaSuccess) return B200GMM_ECUDA;
  if (get != nullptr && (get(&ctx) != CUDA_SUCCESS || ctx == nullptr)) return B200GMM_ECUDA;
  return B200GMM_OK;
}

struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  int pair_ctas = 0;  // CTAs a launch of the 2-CTA-cluster variant may use (even, <= sm_count)
  bool attrs_set = false;
};

// Everything one launch of gmm_kernel needs, whatever the variant.
struct LaunchArgs {
  int grid = 0;
  cudaStream_t stream = nullptr;
  CUtensorMap map_a, map_b, map_b2, map_c, map_a2;
  __nv_bfloat16* c = nullptr;
  const int64_t* batch_sizes = nullptr;  // device
  Problem p;
  uint32_t* status = nullptr;
  CUtensorMap* slots = nullptr;
  uint32_t* sched_counter = nullptr;       // zeroed on the stream before the launch
  const int64_t* row_dest = nullptr;      // scatter / combine epilogue
  const float* row_scale = nullptr;
  int reduce_add = 0;
  const int32_t* a_rows = nullptr;        // gather variant
  const __nv_bfloat16* a_src = nullptr;
  int64_t a_src_rows = 0;
  int64_t dest_lo = 0, dest_hi = 0;       // window every row_dest entry must fall into (0, 0: unchecked)
  const __nv_bfloat16* gate_grad = nullptr;  // gated product: output gradient, selects the backward epilogue
  PushArgs push = {};                     // rows to move while the product runs (src == nullptr: none)
};

template <int MODE, int CTAS, bool GATHER, bool SWIGLU, bool PUSH = false>
cudaError_t launch_gmm(const LaunchArgs& a) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.grid);
  cfg.blockDim = dim3(GATHER ? gather_threads<CTAS, MODE>() : (PUSH ? kGemmPushThreads : kThreads));
  cfg.dynamicSmemBytes = PUSH ? kSmemBytesPush : kSmemBytes;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gmm_kernel<MODE, CTAS, GATHER, SWIGLU, PUSH>, a.map_a, a.map_b, a.map_b2, a.map_c, a.map_a2, a.c,
                            a.batch_sizes, a.p, a.status, a.slots, a.sched_counter, a.row_dest, a.a_rows, a.a_src, a.a_src_rows,
                            a.row_scale, a.reduce_add, a.dest_lo, a.dest_hi, a.gate_grad, a.push);
}

// The plain forward / dgrad kernels with push warps (a.push.src != nullptr).
cudaError_t launch_with_push(const LaunchArgs& a, int ctas) {
  if (a.p.mode == kNN)
    return ctas == 2 ? launch_gmm<kNN, 2, false, false, true>(a) : launch_gmm<kNN, 1, false, false, true>(a);
  if (a.p.mode == kNT)
    return ctas == 2 ? launch_gmm<kNT, 2, false, false, true>(a) : launch_gmm<kNT, 1, false, false, true>(a);
  return cudaErrorInvalidValue;
}

// The layout (a.p.mode) picks the last template argument; the gated product has no wgrad form.
template <int CTAS, bool GATHER, bool SWIGLU>
cudaError_t launch_layout(const LaunchArgs& a) {
  if (a.p.mode == kNN) return launch_gmm<kNN, CTAS, GATHER, SWIGLU>(a);
  if (a.p.mode == kNT) return launch_gmm<kNT, CTAS, GATHER, SWIGLU>(a);
  if constexpr (!SWIGLU) return launch_gmm<kTN, CTAS, GATHER, false>(a);
  return cudaErrorInvalidValue;
}

template <bool GATHER, bool SWIGLU>
cudaError_t launch_variant(const LaunchArgs& a, int ctas) {
  return ctas == 2 ? launch_layout<2, GATHER, SWIGLU>(a) : launch_layout<1, GATHER, SWIGLU>(a);
}

template <int MODE, int CTAS, bool GATHER = false, bool SWIGLU = false, bool PUSH = false>
cudaError_t set_smem_attr() {
  return cudaFuncSetAttribute(gmm_kernel<MODE, CTAS, GATHER, SWIGLU, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(PUSH ? kSmemBytesPush : kSmemBytes));
}

// Per-device facts, looked up once.  Index = CUDA device ordinal.
int device_info(DeviceInfo** out) {
  static std::mutex mu;
  static DeviceInfo infos[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200GMM_ECUDA;
  if (ensure_context(dev) != B200GMM_OK) return B200GMM_ECUDA;
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& d = infos[dev];
  if (d.sm_count == 0) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return B200GMM_ECUDA;
  }
  if (d.cc_major != 10) return B200GMM_EDEVICE;
  if (!d.attrs_set) {
    if (set_smem_attr<kNN, 1>() != cudaSuccess || set_smem_attr<kNT, 1>() != cudaSuccess ||
        set_smem_attr<kTN, 1>() != cudaSuccess || set_smem_attr<kNN, 2>() != cudaSuccess ||
        set_smem_attr<kNT, 2>() != cudaSuccess || set_smem_attr<kTN, 2>() != cudaSuccess ||
        set_smem_attr<kNN, 1, true>() != cudaSuccess || set_smem_attr<kNT, 1, true>() != cudaSuccess ||
        set_smem_attr<kNN, 2, true>() != cudaSuccess || set_smem_attr<kNT, 2, true>() != cudaSuccess ||
        set_smem_attr<kTN, 1, true>() != cudaSuccess || set_smem_attr<kTN, 2, true>() != cudaSuccess ||
        set_smem_attr<kNN, 1, false, true>() != cudaSuccess || set_smem_attr<kNT, 1, false, true>() != cudaSuccess ||
        set_smem_attr<kNN, 2, false, true>() != cudaSuccess || set_smem_attr<kNT, 2, false, true>() != cudaSuccess ||
        set_smem_attr<kNN, 1, false, false, true>() != cudaSuccess || set_smem_attr<kNT, 1, false, false, true>() != cudaSuccess ||
        set_smem_attr<kNN, 2, false, false, true>() != cudaSuccess || set_smem_attr<kNT, 2, false, false, true>() != cudaSuccess)
      return B200GMM_ECUDA;
    // How many 2-CTA clusters of this kernel the device can hold at once (a GPC
    // with an odd number of free SMs leaves one out).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(d.sm_count & ~1);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gmm_kernel<kNN, 2>, &cfg) != cudaSuccess || clusters <= 0) {
      (void)cudaGetLastError();
      clusters = 0;
    }
    d.pair_ctas = 2 * clusters;
    if (d.pair_ctas > (d.sm_count & ~1)) d.pair_ctas = d.sm_count & ~1;
    d.attrs_set = true;
  }
  *out = &d;
  return B200GMM_OK;
}

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return (v != nullptr && *v != '\0') ? std::atoi(v) : fallback;
}

int64_t env_int64(const char* name, int64_t fallback) {
  const char* v = std::getenv(name);
  return (v != nullptr && *v != '\0') ? std::atoll(v) : fallback;
}

// bf16 tensor map (128-byte swizzle unless told otherwise); dims/box innermost first,
// strides in bytes for dimensions 1 .. rank-1 (nullptr: packed).
int encode_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
               const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B,
               const uint64_t* strides = nullptr) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return B200GMM_ECUDA;
  cuuint64_t gdim[4];
  cuuint64_t gstride[3];
  cuuint32_t gbox[4];
  cuuint32_t estride[4] = {1, 1, 1, 1};
  uint64_t stride = 2;
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    stride *= dims[i];
    if (i + 1 < rank) gstride[i] = strides != nullptr ? strides[i] : stride;
  }
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank),
                        const_cast<void*>(base), gdim, gstride, gbox, estride,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS && env_int("B200GMM_DEBUG", 0) != 0) {
    std::fprintf(stderr, "b200gmm: cuTensorMapEncodeTiled -> %d: base %p rank %d dims {%llu,%llu,%llu} box {%u,%u,%u}\n",
                 static_cast<int>(r), base, rank, (unsigned long long)gdim[0], (unsigned long long)gdim[1],
                 (unsigned long long)(rank > 2 ? gdim[2] : 0), gbox[0], gbox[1], rank > 2 ? gbox[2] : 0u);
  }
  return r == CUDA_SUCCESS ? B200GMM_OK : B200GMM_ETENSORMAP;
}

// A row-major [.., rows, cols] operand whose tiles are staged as boxes of 64 columns
// (MN-major for the tensor core): seen as {64, rows, cols / 64 (, experts)}, one TMA
// load brings `boxes` neighbouring 64-column boxes, which land one after the other
// in shared memory exactly as separate loads would put them.  cols % 64 == 0.
int encode_blocked(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t experts,
                   uint32_t box_rows, uint32_t boxes) {
  const uint64_t dims[4] = {64, rows, cols / 64, experts};
  const uint64_t strides[3] = {cols * 2, 128, rows * cols * 2};
  const uint32_t box[4] = {64, box_rows, boxes, 1};
  return encode_map(map, base, experts > 0 ? 4 : 3, dims, box, CU_TENSOR_MAP_SWIZZLE_128B, strides);
}

// Which variant a problem runs on.  Only shapes known on the host may decide
// (batch_sizes can live on the device): a CTA pair pays off when an expert has,
// on average, at least a couple of 256-row tiles.  B200GMM_CTAS=1|2 overrides.
int choose_ctas(int z, int64_t tokens, int64_t d1, int trans_a) {
  const int forced = env_int("B200GMM_CTAS", 0);
  if (forced == 1 || forced == 2) return forced;
  if (z <= 0 || tokens / z < 512) return 1;
  return (!trans_a || d1 >= 256) ? 2 : 1;
}

// Which kernel features a plain, gathered or gated launch uses (schedule.cuh: Problem).
struct Features {
  bool gather = false;
  bool swiglu = false;
};

int check_problem(int z, int64_t tokens, int64_t d1, int64_t n, int trans_a, int trans_b, int ctas,
                  Problem* p, const Features& f = Features()) {
  if (trans_a && trans_b) return B200GMM_EINVAL;
  if (z < 0 || tokens < 0 || d1 < 0 || n < 0) return B200GMM_EINVAL;
  if (z > kMaxExperts) return B200GMM_ELIMIT;
  if ((d1 % 8) != 0 || (n % 8) != 0) return B200GMM_EALIGN;
  if (tokens >= (int64_t(1) << 31) - 256 || d1 >= (int64_t(1) << 31) - 256 ||
      n >= (int64_t(1) << 31) - 256)
    return B200GMM_ELIMIT;
  p->mode = trans_a ? kTN : (trans_b ? kNT : kNN);
  p->z = z;
  p->tokens = tokens;
  p->d1 = d1;
  p->n = n;
  if (ctas != 1 && ctas != 2) return B200GMM_EINVAL;
  p->tile_m = kBlockM * ctas;
  derive(p);
  p->wide_a = 0;
  p->wide_b = 0;
  p->group_m = env_int("B200GMM_GROUP_M", ctas == 2 ? 8 : 16);
  if (p->group_m < 1) p->group_m = 1;
  // Tiles are drawn from a global counter.  For wgrad, where a tile's duration is
  // its expert's row count, the experts are taken largest first, so that the
  // CTAs that finish early find short tiles left.
  p->order = (z > 1 && p->mode == kTN) ? 1 : 0;
  // Transposed tiles for experts of at most 64 rows: off unless asked for.  They
  // take 4x fewer tensor-core cycles on such experts, but those experts are bound
  // by streaming their weights from HBM either way, and measured end to end the
  // launch was not faster with them (B200GMM_LIGHT=1 switches them on).
  p->light = (p->mode != kTN && ctas == 1 && !f.gather && !f.swiglu) ? env_int("B200GMM_LIGHT", 0) : 0;
  const int64_t wait_ns = env_int64("B200GMM_WAIT_LIMIT_NS", static_cast<int64_t>(ptx::kWaitLimitNs));
  p->wait_ns = wait_ns > 0 ? wait_ns : static_cast<int64_t>(ptx::kWaitLimitNs);
  // Upper bound on the tile count must fit the kernel's 32-bit tile index (twice:
  // positions drawn past the end still have to fit).
  const int64_t nt = (n + kBlockN - 1) / kBlockN;
  const int64_t row_tiles = trans_a ? int64_t(z) * ((d1 + p->tile_m - 1) / p->tile_m)
                                    : (tokens / p->tile_m + 3 * int64_t(z));  // + transposed tiles, half as wide
  if (row_tiles * nt >= (int64_t(1) << 30)) return B200GMM_ELIMIT;
  return B200GMM_OK;
}

// Argument checks alone (no launch): what run_impl would refuse for these sizes.
int check_args_only(int z, int64_t tokens, int64_t d1, int64_t n, int trans_b) {
  Problem p;
  return check_problem(z, tokens, d1, n, 0, trans_b, 1, &p);
}

size_t round128(size_t x) { return (x + 127) & ~size_t(127); }

// ---- scratch for b200gmm_run_static ------------------------------------------
// Same layout as a caller-provided workspace, sized for the entry point's own
// expert limit.  Lives in every CUDA context that loads this library, from load
// until exit.
constexpr size_t kStaticScratchBytes =
    ((size_t(B200GMM_STATIC_MAX_EXPERTS) * sizeof(int64_t) + 16 + 127) & ~size_t(127)) +
    size_t(kMaxCtas) * kMapSlots * 2 * sizeof(CUtensorMap);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device.  In host code the
// symbol's name is only a handle; the address a kernel can use has to be asked
// for, per device, with that device current.
int static_scratch_address(void** out) {
  // One lookup per device; afterwards a plain atomic load, no lock.
  static std::atomic<void*> addr[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200GMM_ECUDA;
  void* p = addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    std::lock_guard<std::mutex> lock(mu);
    p = addr[dev].load(std::memory_order_relaxed);
    if (p == nullptr) {
      if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
        (void)cudaGetLastError();
        return B200GMM_ECUDA;
      }
      addr[dev].store(p, std::memory_order_release);
    }
  }
  *out = p;
  return B200GMM_OK;
}

// Workspace layout: [0, 8z) device copy of batch_sizes; then, 128-byte aligned,
// kMaxCtas x kMapSlots x {a, b} tensor maps edited by the wgrad kernel.
size_t maps_offset(int z) { return round128(size_t(z) * sizeof(int64_t) + 16); }
size_t maps_bytes() { return size_t(kMaxCtas) * kMapSlots * 2 * sizeof(CUtensorMap); }

}  // namespace

extern "C" {

int b200gmm_workspace_bytes(int z, size_t* out_bytes) {
  if (out_bytes == nullptr || z < 0) return B200GMM_EINVAL;
  if (z > kMaxExperts) return B200GMM_ELIMIT;
  *out_bytes = maps_offset(z) + maps_bytes();
  return B200GMM_OK;
}

}  // extern "C"

namespace {

// Shared body of b200gmm_run and b200gmm_run_scatter.  row_dest == nullptr: rows
// go to c.  Otherwise (non-transposed a only) row i of the result goes to the
// address row_dest[i] and c is not touched.
int run_impl(const void* a, const void* b, void* c, const int64_t* batch_sizes,
             int batch_sizes_on_device, int z, int64_t tokens, int64_t dim_a1, int64_t n,
             int trans_a, int trans_b, void* workspace, size_t workspace_bytes,
             uint32_t* device_status, void* cuda_stream, const int64_t* row_dest,
             const int32_t* a_rows = nullptr, int64_t a_source_rows = 0, const void* b2 = nullptr,
             const float* row_scale = nullptr, int reduce_add = 0, const void* dest_base = nullptr,
             int64_t dest_bytes = 0, const void* gate_grad = nullptr, const PushArgs* push = nullptr,
             bool* push_launched = nullptr) {
  // push != nullptr: rows to move inside the same launch (plain forward / dgrad
  // kernels only); *push_launched tells the caller whether a launch took them.
  // gate_grad != nullptr: backward epilogue of the gated product; c is [2, tokens, n].
  if (gate_grad != nullptr && (b2 == nullptr || row_dest != nullptr || (reinterpret_cast<uintptr_t>(gate_grad) & 15)))
    return B200GMM_EINVAL;
  if (dest_base != nullptr && (row_dest == nullptr || dest_bytes < 0)) return B200GMM_EINVAL;
  if ((row_scale != nullptr || reduce_add) && row_dest == nullptr) return B200GMM_EINVAL;
  if (a_rows != nullptr && (dim_a1 == 0 || a_source_rows <= 0 || (trans_a && row_dest != nullptr)))
    return B200GMM_EINVAL;
  // b2 != nullptr: gated product silu(a @ b) * (a @ b2); n counts the columns of
  // each of b, b2 and c, the schedule runs over 2n virtual columns.
  const bool swiglu = (b2 != nullptr);
  if (swiglu && (trans_a || a_rows != nullptr)) return B200GMM_EINVAL;
  if (swiglu && (reinterpret_cast<uintptr_t>(b2) & 15)) return B200GMM_EALIGN;
  if (swiglu && (n % 8) != 0) return B200GMM_EALIGN;
  const int64_t n_out = n;
  if (swiglu) n = 2 * n;
  if (row_dest != nullptr) {
    if (trans_a || dim_a1 == 0) return B200GMM_EINVAL;
    if (c == nullptr) c = const_cast<void*>(a);  // never written; keeps the argument checks below uniform
  }
  Problem p;
  Features feat;
  feat.gather = (a_rows != nullptr);
  feat.swiglu = swiglu;
  int ctas = choose_ctas(z, tokens, dim_a1, trans_a);
  int rc = check_problem(z, tokens, dim_a1, n, trans_a, trans_b, ctas, &p, feat);
  if (rc != B200GMM_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (z == 0) return B200GMM_OK;
  if (batch_sizes == nullptr) return B200GMM_EINVAL;

  // Degenerate shapes: nothing to multiply.  Only wgrad has output to define
  // (zeros), and only when that output is non-empty.
  if (p.mode == kTN) {
    if (dim_a1 == 0 || n == 0) return B200GMM_OK;
    if (c == nullptr) return B200GMM_EINVAL;
    if (tokens == 0) {
      if (cudaMemsetAsync(c, 0, size_t(z) * size_t(dim_a1) * size_t(n) * 2, stream) != cudaSuccess)
        return B200GMM_ECUDA;
      return B200GMM_OK;
    }
  } else {
    if (tokens == 0 || n == 0) return B200GMM_OK;
    if (c == nullptr) return B200GMM_EINVAL;
    if (dim_a1 == 0) {
      // k == 0: every product is an empty sum.
      if (cudaMemsetAsync(c, 0, size_t(tokens) * size_t(n_out) * 2, stream) != cudaSuccess)
        return B200GMM_ECUDA;
      return B200GMM_OK;
    }
  }
  if (a == nullptr || b == nullptr) return B200GMM_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
      (reinterpret_cast<uintptr_t>(c) & 15))
    return B200GMM_EALIGN;

  DeviceInfo* dev = nullptr;
  rc = device_info(&dev);
  if (rc != B200GMM_OK) return rc;

  if (ctas == 2 && dev->pair_ctas < 2) {
    ctas = 1;
    if ((rc = check_problem(z, tokens, dim_a1, n, trans_a, trans_b, ctas, &p, feat)) != B200GMM_OK) return rc;
  }

  size_t need = 0;
  b200gmm_workspace_bytes(z, &need);
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 127))
    return B200GMM_EWORKSPACE;
  CUtensorMap* slots = reinterpret_cast<CUtensorMap*>(static_cast<char*>(workspace) + maps_offset(z));
  // The tile counter of the kernel's scheduler sits in the 16 bytes after the
  // batch_sizes copy and starts every launch at zero.
  uint32_t* sched_counter = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + size_t(z) * sizeof(int64_t));
  if (cudaMemsetAsync(sched_counter, 0, 16, stream) != cudaSuccess) return B200GMM_ECUDA;

  const int64_t* bs_dev = batch_sizes;
  if (!batch_sizes_on_device) {
    if (cudaMemcpyAsync(workspace, batch_sizes, size_t(z) * sizeof(int64_t), cudaMemcpyHostToDevice,
                        stream) != cudaSuccess)
      return B200GMM_ECUDA;
    bs_dev = static_cast<const int64_t*>(workspace);
  }

  CUtensorMap map_a, map_b, map_b2, map_a2;
  bool have_b2 = swiglu;
  // N: columns of b (and of b2, and of c); the Problem's n is twice that for the gated product.
  const uint64_t T = uint64_t(tokens), D1 = uint64_t(dim_a1), N = uint64_t(n_out), Z = uint64_t(z);
  const bool gather = (a_rows != nullptr);  // a is then fetched row by row, without a tensor map
  if (p.mode == kNN) {
    const uint64_t da[2] = {D1, T};
    const uint32_t ba[2] = {kBlockK, uint32_t(kBlockM)};
    const uint64_t db[3] = {N, D1, Z};
    const uint32_t bb[3] = {64, kBlockK, 1};
    // (One load per 64-column box: a single load of all the boxes of a stage through
    // a {64, k, n / 64, z} view of b measured 10-15 % slower in this layout.)
    if ((rc = encode_map(&map_b, b, 3, db, bb)) != 0) return rc;
    if (swiglu && (rc = encode_map(&map_b2, b2, 3, db, bb)) != 0) return rc;
    if (gather) map_a = map_b;
    else if ((rc = encode_map(&map_a, a, 2, da, ba)) != 0) return rc;
    if (p.light) {  // transposed tiles fetch their few rows of a in boxes of 32
      const uint32_t bl[2] = {kBlockK, 32};
      if ((rc = encode_map(&map_a2, a, 2, da, bl)) != 0) return rc;
    }
  } else if (p.mode == kNT) {
    const uint64_t da[2] = {D1, T};
    const uint32_t ba[2] = {kBlockK, uint32_t(kBlockM)};
    const uint64_t db[3] = {D1, N, Z};
    // rows of b per box: a CTA's share of the tile; for the gated product half a tile from each of b, b2
    const uint32_t bb[3] = {kBlockK, uint32_t(swiglu ? kBlockN / 2 : kBlockN / ctas), 1};
    if ((rc = encode_map(&map_b, b, 3, db, bb)) != 0) return rc;
    if (swiglu && (rc = encode_map(&map_b2, b2, 3, db, bb)) != 0) return rc;
    if (gather) map_a = map_b;
    else if ((rc = encode_map(&map_a, a, 2, da, ba)) != 0) return rc;
    if (p.light) {  // transposed tiles: rows of a in boxes of 32, 128 rows of b[i] as the M operand
      const uint32_t bl[2] = {kBlockK, 32};
      const uint32_t bw[3] = {kBlockK, uint32_t(kLightCols), 1};
      if ((rc = encode_map(&map_a2, a, 2, da, bl)) != 0) return rc;
      if ((rc = encode_map(&map_b2, b, 3, db, bw)) != 0) return rc;
      have_b2 = true;
    }
  } else {
    const uint64_t da[2] = {D1, T};
    const uint64_t db[2] = {N, T};
    const uint32_t bx[2] = {64, kBlockK};
    // wgrad: both operands are staged as 64-column boxes; where the column count
    // allows, one load brings all boxes of a stage (half the TMA instructions).
    p.wide_b = (N % 64 == 0) ? 1 : 0;
    p.wide_a = (D1 % 64 == 0 && !gather) ? 1 : 0;
    if (p.wide_b) rc = encode_blocked(&map_b, b, N, T, 0, kBlockK, kBlockN / ctas / 64);
    else rc = encode_map(&map_b, b, 2, db, bx);
    if (rc != 0) return rc;
    if (gather) map_a = map_b;
    else if ((rc = p.wide_a ? encode_blocked(&map_a, a, D1, T, 0, kBlockK, kBlockM / 64)
                            : encode_map(&map_a, a, 2, da, bx)) != 0) return rc;
  }

  if (!have_b2) map_b2 = map_b;  // unused by the kernel, but a valid map
  if (!p.light) map_a2 = map_a;

  // Output map for the epilogue's TMA stores: 32 x 32 boxes, 64-byte swizzle; for
  // wgrad, whose c[z, m, n] is addressed as z*m rows, 64 x 32 boxes with 128-byte
  // swizzle.  Unused (left zeroed) when the rows are scattered through row_dest.
  CUtensorMap map_c = {};
  if (row_dest == nullptr) {
    const uint64_t dc[2] = {N, p.mode == kTN ? Z * D1 : (gate_grad != nullptr ? 2 * T : T)};
    const uint32_t bc[2] = {p.mode == kTN ? 64u : 32u, 32};
    if (dc[1] >= (uint64_t(1) << 31)) return B200GMM_ELIMIT;
    if ((rc = encode_map(&map_c, c, 2, dc, bc, p.mode == kTN ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B)) != 0)
      return rc;
  }

  LaunchArgs la;
  const int max_grid = (ctas == 2) ? dev->pair_ctas : dev->sm_count;
  la.grid = max_grid < kMaxCtas ? max_grid : kMaxCtas;
  la.stream = stream;
  la.map_a = map_a;
  la.map_b = map_b;
  la.map_b2 = map_b2;
  la.map_c = map_c;
  la.map_a2 = map_a2;
  la.sched_counter = sched_counter;
  la.c = static_cast<__nv_bfloat16*>(c);
  la.batch_sizes = bs_dev;
  la.p = p;
  la.status = device_status;
  la.slots = slots;
  la.row_dest = row_dest;
  la.row_scale = row_scale;
  la.reduce_add = reduce_add;
  la.gate_grad = static_cast<const __nv_bfloat16*>(gate_grad);
  if (dest_base != nullptr) {
    la.dest_lo = static_cast<int64_t>(reinterpret_cast<uintptr_t>(dest_base));
    la.dest_hi = la.dest_lo + dest_bytes;
    if (la.dest_hi == 0) la.dest_hi = 1;  // an empty window at address 0 still rejects every row
  }
  if (gather) {
    la.a_rows = a_rows;
    la.a_src = static_cast<const __nv_bfloat16*>(a);
    la.a_src_rows = a_source_rows;
  }
  const bool with_push = push != nullptr && push->src != nullptr && push->n_items > 0 && !gather && !swiglu &&
                         p.mode != kTN;
  if (with_push) {
    la.push = *push;
    la.push.via_tma = env_int("B200GMM_PUSH_TMA", 1) ? 1 : 0;  // bulk copies measured faster than the register path
    // Optional pacing: spread the transfer over a share (B200GMM_PUSH_SPREAD percent; default
    // 0, as fast as it goes, which measured best) of the time the product is expected to
    // take at 1 PFLOP/s.
    const int spread = env_int("B200GMM_PUSH_SPREAD", 0);
    const double product_ns = 2.0 * double(tokens) * double(dim_a1) * double(n) / 1.0e6;
    const int64_t warps = int64_t(la.grid) * kPushWarps;
    const int64_t items_per_warp = (push->n_items + warps - 1) / warps;
    la.push.interval_ns = (spread > 0 && items_per_warp > 0)
                              ? static_cast<int64_t>(product_ns * (spread > 100 ? 100 : spread) / 100.0 / double(items_per_warp))
                              : 0;
    // (the pacing is a wait like any other: all of it stays inside the wait limit)
    if (la.push.interval_ns * items_per_warp > p.wait_ns) la.push.interval_ns = p.wait_ns / items_per_warp;
  }
  const cudaError_t err = gather      ? launch_variant<true, false>(la, ctas)
                          : swiglu    ? launch_variant<false, true>(la, ctas)
                          : with_push ? launch_with_push(la, ctas)
                                      : launch_variant<false, false>(la, ctas);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return B200GMM_ECUDA;
  }
  if (with_push && push_launched != nullptr) *push_launched = true;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200GMM_OK;
}

}  // namespace

extern "C" {

int b200gmm_run(const void* a, const void* b, void* c, const int64_t* batch_sizes,
                int batch_sizes_on_device, int z, int64_t tokens, int64_t dim_a1, int64_t n,
                int trans_a, int trans_b, void* workspace, size_t workspace_bytes,
                uint32_t* device_status, void* cuda_stream) {
  return run_impl(a, b, c, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, trans_a, trans_b,
                  workspace, workspace_bytes, device_status, cuda_stream, nullptr);
}

int b200gmm_run_scatter(const void* a, const void* b, const int64_t* row_dest, const void* dest_base,
                        int64_t dest_bytes, const int64_t* batch_sizes,
                        int batch_sizes_on_device, int z, int64_t tokens, int64_t dim_a1, int64_t n,
                        int trans_b, void* workspace, size_t workspace_bytes, uint32_t* device_status,
                        void* cuda_stream) {
  if (row_dest == nullptr) return B200GMM_EINVAL;
  return run_impl(a, b, nullptr, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, 0, trans_b,
                  workspace, workspace_bytes, device_status, cuda_stream, row_dest, nullptr, 0, nullptr, nullptr, 0,
                  dest_base, dest_bytes);
}

int b200gmm_run_scatter_push(const void* a, const void* b, const int64_t* row_dest, const void* dest_base,
                             int64_t dest_bytes, const int64_t* batch_sizes, int batch_sizes_on_device, int z,
                             int64_t tokens, int64_t dim_a1, int64_t n, int trans_b, const void* push_src,
                             int64_t push_row_bytes, int64_t push_items, const int32_t* push_src_row,
                             const int32_t* push_dst_rank, const int64_t* push_dst_row,
                             const void* const* push_peer_base, void* workspace, size_t workspace_bytes,
                             uint32_t* device_status, void* cuda_stream) {
  if (row_dest == nullptr) return B200GMM_EINVAL;
  if (push_row_bytes <= 0 || (push_row_bytes % 16) != 0 || push_items < 0) return B200GMM_EINVAL;
  if (push_items > 0) {
    if (push_src == nullptr || push_dst_rank == nullptr || push_dst_row == nullptr || push_peer_base == nullptr)
      return B200GMM_EINVAL;
    if (reinterpret_cast<uintptr_t>(push_src) & 15) return B200GMM_EALIGN;
  }
  PushArgs push = {};
  push.src = static_cast<const uint4*>(push_src);
  push.row_vecs = push_row_bytes / 16;
  push.n_items = push_items;
  push.src_row = push_src_row;
  push.dst_rank = push_dst_rank;
  push.dst_row = push_dst_row;
  push.peer_base = const_cast<void* const*>(push_peer_base);
  push.interval_ns = 0;
  push.via_tma = 0;
  bool pushed = false;
  const int rc = run_impl(a, b, nullptr, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, 0, trans_b,
                          workspace, workspace_bytes, device_status, cuda_stream, row_dest, nullptr, 0, nullptr,
                          nullptr, 0, dest_base, dest_bytes, nullptr, &push, &pushed);
  if (rc != B200GMM_OK || pushed || push_items == 0) return rc;
  // The product was empty and launched nothing: the rows still have to move.
  return b200gmm_push_rows(push_src, push_row_bytes, push_items, push_src_row, push_dst_rank, push_dst_row,
                           push_peer_base, 0, cuda_stream);
}

int b200gmm_run_combine(const void* a, const void* b, const int64_t* row_dest, const void* dest_base,
                        int64_t dest_bytes, const float* row_weight,
                        int accumulate, const int64_t* batch_sizes, int batch_sizes_on_device, int z,
                        int64_t tokens, int64_t dim_a1, int64_t n, int trans_b, void* workspace,
                        size_t workspace_bytes, uint32_t* device_status, void* cuda_stream) {
  if (row_dest == nullptr) return B200GMM_EINVAL;
  if (row_weight != nullptr && (reinterpret_cast<uintptr_t>(row_weight) & 3)) return B200GMM_EALIGN;
  // k == 0 would take the zero-fill shortcut of the shared body, which writes c;
  // a combine has no c, and adding zeros changes nothing.
  if (dim_a1 == 0) return accumulate ? B200GMM_OK : B200GMM_EINVAL;
  return run_impl(a, b, nullptr, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, 0, trans_b,
                  workspace, workspace_bytes, device_status, cuda_stream, row_dest, nullptr, 0, nullptr,
                  row_weight, accumulate ? 1 : 0, dest_base, dest_bytes);
}

int b200gmm_run_gather(const void* x, int64_t x_rows, const int32_t* row_index, const void* b, void* c,
                       const int64_t* row_dest, const void* dest_base, int64_t dest_bytes,
                       const int64_t* batch_sizes, int batch_sizes_on_device,
                       int z, int64_t tokens, int64_t dim_a1, int64_t n, int trans_b, void* workspace,
                       size_t workspace_bytes, uint32_t* device_status, void* cuda_stream) {
  if (row_index == nullptr || x_rows <= 0 || x_rows >= (int64_t(1) << 31)) return B200GMM_EINVAL;
  if (c == nullptr && row_dest == nullptr) return B200GMM_EINVAL;
  return run_impl(x, b, c, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, 0, trans_b, workspace,
                  workspace_bytes, device_status, cuda_stream, row_dest, row_index, x_rows, nullptr, nullptr, 0,
                  dest_base, dest_bytes);
}

int b200gmm_run_gather_wgrad(const void* x, int64_t x_rows, const int32_t* row_index, const void* grad, void* c,
                             const int64_t* batch_sizes, int batch_sizes_on_device, int z, int64_t tokens,
                             int64_t dim_x1, int64_t n, void* workspace, size_t workspace_bytes,
                             uint32_t* device_status, void* cuda_stream) {
  if (row_index == nullptr || x_rows <= 0 || x_rows >= (int64_t(1) << 31)) return B200GMM_EINVAL;
  return run_impl(x, grad, c, batch_sizes, batch_sizes_on_device, z, tokens, dim_x1, n, 1, 0, workspace,
                  workspace_bytes, device_status, cuda_stream, nullptr, row_index, x_rows);
}

int b200gmm_run_swiglu(const void* a, const void* b_gate, const void* b_up, void* c, const int64_t* row_dest,
                       const void* dest_base, int64_t dest_bytes, const int64_t* batch_sizes, int batch_sizes_on_device, int z, int64_t tokens,
                       int64_t dim_a1, int64_t n, int trans_b, void* workspace, size_t workspace_bytes,
                       uint32_t* device_status, void* cuda_stream) {
  if (c == nullptr && row_dest == nullptr) return B200GMM_EINVAL;
  if (b_up == nullptr && tokens > 0 && n > 0 && dim_a1 > 0 && z > 0) return B200GMM_EINVAL;
  if (b_up == nullptr || dim_a1 == 0)  // nothing to multiply: silu(0) * 0 = 0, the plain path's zeros
    return run_impl(a, b_gate, c, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, 0, trans_b, workspace,
                    workspace_bytes, device_status, cuda_stream, row_dest, nullptr, 0, nullptr, nullptr, 0, dest_base,
                    dest_bytes);
  return run_impl(a, b_gate, c, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, 0, trans_b, workspace,
                  workspace_bytes, device_status, cuda_stream, row_dest, nullptr, 0, b_up, nullptr, 0, dest_base,
                  dest_bytes);
}

int b200gmm_run_swiglu_backward(const void* a, const void* b_gate, const void* b_up, const void* grad_out,
                                void* grad_products, const int64_t* batch_sizes, int batch_sizes_on_device, int z,
                                int64_t tokens, int64_t dim_a1, int64_t n, int trans_b, void* workspace,
                                size_t workspace_bytes, uint32_t* device_status, void* cuda_stream) {
  if (grad_products == nullptr || (grad_out == nullptr && tokens > 0 && n > 0)) return B200GMM_EINVAL;
  if (b_up == nullptr && tokens > 0 && n > 0 && dim_a1 > 0 && z > 0) return B200GMM_EINVAL;
  if (dim_a1 == 0 || tokens == 0 || n == 0 || z == 0) {
    // g = u = 0 everywhere: dg = dh * 0 * silu'(0) = 0 and du = dh * silu(0) = 0
    if (tokens > 0 && n > 0 && z > 0 &&
        cudaMemsetAsync(grad_products, 0, size_t(2) * size_t(tokens) * size_t(n) * 2,
                        static_cast<cudaStream_t>(cuda_stream)) != cudaSuccess)
      return B200GMM_ECUDA;
    return check_args_only(z, tokens, dim_a1, n, trans_b);
  }
  return run_impl(a, b_gate, grad_products, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, 0, trans_b,
                  workspace, workspace_bytes, device_status, cuda_stream, nullptr, nullptr, 0, b_up, nullptr, 0, nullptr, 0,
                  grad_out);
}

int b200gmm_run_static(const void* a, const void* b, void* c, const int64_t* batch_sizes,
                       int batch_sizes_on_device, int z, int64_t tokens, int64_t dim_a1, int64_t n,
                       int trans_a, int trans_b, uint32_t* device_status, void* cuda_stream) {
  if (z > B200GMM_STATIC_MAX_EXPERTS) return B200GMM_ELIMIT;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != B200GMM_OK) return rc;
  return b200gmm_run(a, b, c, batch_sizes, batch_sizes_on_device, z, tokens, dim_a1, n, trans_a,
                     trans_b, scratch, kStaticScratchBytes, device_status, cuda_stream);
}

int b200gmm_push_rows(const void* src, int64_t row_bytes, int64_t n_items, const int32_t* src_row,
                      const int32_t* dst_rank, const int64_t* dst_row, const void* const* peer_base,
                      int max_ctas, void* cuda_stream) {
  if (row_bytes <= 0 || (row_bytes % 16) != 0 || n_items < 0) return B200GMM_EINVAL;
  if (n_items == 0) return B200GMM_OK;
  if (src == nullptr || dst_rank == nullptr || dst_row == nullptr || peer_base == nullptr)
    return B200GMM_EINVAL;
  if (reinterpret_cast<uintptr_t>(src) & 15) return B200GMM_EALIGN;
  DeviceInfo* dev = nullptr;
  const int rc = device_info(&dev);
  if (rc != B200GMM_OK) return rc;
  // Rows are handed out grid-stride to 4 CTAs per SM: enough loads in flight to
  // fill NVLink and HBM.  max_ctas > 0 caps the grid for a transfer that should
  // leave memory bandwidth to other work.
  int64_t grid = int64_t(dev->sm_count) * 4;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid > n_items) grid = n_items;
  push_rows_kernel<<<static_cast<unsigned>(grid), kPushThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(src), row_bytes / 16, n_items, src_row, dst_rank, dst_row,
      const_cast<void* const*>(peer_base));
  if (cudaGetLastError() != cudaSuccess) return B200GMM_ECUDA;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200GMM_OK;
}

int b200gmm_sum_slots(const void* slots, void* out, int64_t tokens, int top_k, int64_t cols, void* cuda_stream) {
  if (tokens < 0 || cols < 0 || top_k < 1 || top_k > kSumMaxTopK || (cols % 8) != 0) return B200GMM_EINVAL;
  if (tokens == 0 || cols == 0) return B200GMM_OK;
  if (slots == nullptr || out == nullptr) return B200GMM_EINVAL;
  if ((reinterpret_cast<uintptr_t>(slots) | reinterpret_cast<uintptr_t>(out)) & 15) return B200GMM_EALIGN;
  DeviceInfo* dev = nullptr;
  const int rc = device_info(&dev);
  if (rc != B200GMM_OK) return rc;
  const int64_t total = tokens * (cols / 8);
  int64_t grid = (total + kSumThreads - 1) / kSumThreads;
  const int64_t cap = int64_t(dev->sm_count) * 16;
  if (grid > cap) grid = cap;
  sum_slots_kernel<<<static_cast<unsigned>(grid), kSumThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(slots), static_cast<uint4*>(out), tokens, top_k, cols / 8);
  if (cudaGetLastError() != cudaSuccess) return B200GMM_ECUDA;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200GMM_OK;
}

int b200gmm_fill_offsets(const int64_t* batch_sizes_device, int z, int64_t dim_a1, int64_t n,
                         int trans_a, int trans_b, int64_t* out_device, void* cuda_stream) {
  if (trans_a && trans_b) return B200GMM_EINVAL;
  if (z < 0 || dim_a1 < 0 || n < 0) return B200GMM_EINVAL;
  if (z > kMaxExperts) return B200GMM_ELIMIT;
  if (z == 0) return B200GMM_OK;
  if (batch_sizes_device == nullptr || out_device == nullptr) return B200GMM_EINVAL;
  Problem p = {};
  p.mode = trans_a ? kTN : (trans_b ? kNT : kNN);
  p.z = z;
  p.d1 = dim_a1;
  p.n = n;
  p.tile_m = kBlockM;
  p.group_m = 1;
  derive(&p);
  fill_offsets_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(batch_sizes_device, p,
                                                                            out_device);
  if (cudaGetLastError() != cudaSuccess) return B200GMM_ECUDA;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200GMM_OK;
}

int b200gmm_schedule_host(const int64_t* batch_sizes_host, int z, int64_t tokens, int64_t dim_a1,
                          int64_t n, int trans_a, int trans_b, int cluster_ctas, int64_t* out,
                          int64_t max_tiles, int64_t* n_tiles) {
  Problem p;
  if (cluster_ctas == 0) cluster_ctas = choose_ctas(z, tokens, dim_a1, trans_a);
  const int rc = check_problem(z, tokens, dim_a1, n, trans_a, trans_b, cluster_ctas, &p);
  if (rc != B200GMM_OK) return rc;
  if (n_tiles == nullptr || (z > 0 && batch_sizes_host == nullptr)) return B200GMM_EINVAL;
  // The kernels' build_schedule, replayed: clamped row prefix sums, the order of
  // the experts, tile prefix sums in that order.
  std::vector<int> row_start(size_t(z) + 1), perm(static_cast<size_t>(z)), tile_start(size_t(z) + 1);
  int64_t start = 0;
  for (int e = 0; e < z; ++e) {
    row_start[e] = static_cast<int>(start < tokens ? start : tokens);
    start += batch_sizes_host[e] < 0 ? 0 : batch_sizes_host[e];
  }
  row_start[z] = static_cast<int>(start < tokens ? start : tokens);
  for (int e = 0; e < z; ++e) perm[e] = e;
  if (p.order)
    std::stable_sort(perm.begin(), perm.end(), [&](int x, int y) {
      return row_start[x + 1] - row_start[x] > row_start[y + 1] - row_start[y];
    });
  tile_start[0] = 0;
  for (int i = 0; i < z; ++i)
    tile_start[i + 1] = tile_start[i] + expert_tiles(p, row_start[perm[i] + 1] - row_start[perm[i]]);
  const int total = tile_start[z];
  int pos = 0;
  for (int t = 0; t < total && out != nullptr && t < max_tiles; ++t) {
    while (t >= tile_start[pos + 1]) ++pos;
    const int e = perm[pos];
    const Tile tile = make_tile(p, e, t - tile_start[pos], row_start[e], row_start[e + 1]);
    int64_t* o = out + int64_t(t) * B200GMM_SCHEDULE_FIELDS;
    o[0] = tile.expert;
    o[1] = tile.row0;
    o[2] = tile.col0;
    o[3] = tile.valid_rows;
    o[4] = tile_stages(tile);
    o[5] = tile.kind;
  }
  *n_tiles = total;
  return B200GMM_OK;
}

int b200gmm_schedule_device(const int64_t* batch_sizes_device, int z, int64_t tokens, int64_t dim_a1,
                            int64_t n, int trans_a, int trans_b, int cluster_ctas, int32_t* out_device,
                            int64_t max_tiles, int32_t* n_tiles_device, uint32_t* device_status,
                            void* cuda_stream) {
  Problem p;
  if (cluster_ctas == 0) cluster_ctas = choose_ctas(z, tokens, dim_a1, trans_a);
  const int rc = check_problem(z, tokens, dim_a1, n, trans_a, trans_b, cluster_ctas, &p);
  if (rc != B200GMM_OK) return rc;
  if (n_tiles_device == nullptr || (z > 0 && batch_sizes_device == nullptr) || max_tiles < 0 ||
      max_tiles >= (int64_t(1) << 31) || (max_tiles > 0 && out_device == nullptr))
    return B200GMM_EINVAL;
  schedule_dump_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      batch_sizes_device, p, out_device, static_cast<int>(max_tiles), n_tiles_device, device_status);
  if (cudaGetLastError() != cudaSuccess) return B200GMM_ECUDA;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200GMM_OK;
}

int b200gmm_selftest_wait_timeout(int64_t limit_ns, uint32_t* device_status, void* cuda_stream) {
  // A limit beyond a tenth of a second would only hold the GPU for nothing.
  if (limit_ns <= 0 || limit_ns > 100000000 || device_status == nullptr) return B200GMM_EINVAL;
  wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(static_cast<uint64_t>(limit_ns),
                                                                           device_status);
  if (cudaGetLastError() != cudaSuccess) return B200GMM_ECUDA;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200GMM_OK;
}

int b200gmm_tile_shape(int cluster_ctas, int* out3) {
  if (out3 == nullptr || (cluster_ctas != 1 && cluster_ctas != 2)) return B200GMM_EINVAL;
  out3[0] = kBlockM * cluster_ctas;
  out3[1] = kBlockN;
  out3[2] = kBlockK;
  return B200GMM_OK;
}

int64_t b200gmm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* b200gmm_strerror(int code) {
  switch (code) {
    case B200GMM_OK: return "ok";
    case B200GMM_EINVAL: return "invalid argument (null pointer, negative size, or trans_a and trans_b both set)";
    case B200GMM_EALIGN: return "row lengths must be multiples of 8 bf16 elements and pointers 16-byte aligned";
    case B200GMM_ELIMIT: return "too many experts (max 1024), too many tiles, or a dimension >= 2^31";
    case B200GMM_EWORKSPACE: return "workspace missing, smaller than b200gmm_workspace_bytes(z), or not 128-byte aligned";
    case B200GMM_ECUDA: return "a CUDA runtime or driver call failed";
    case B200GMM_ETENSORMAP: return "cuTensorMapEncodeTiled rejected a tensor (address, stride or extent)";
    case B200GMM_EDEVICE: return "current device is not compute capability 10.x (B200, sm_100a)";
    case B200GMM_ETIMEOUT: return "a bounded wait inside the kernel gave up (device status word)";
    default: return "unknown b200gmm error code";
  }
}

}  // extern "C"
