/*
 * b200gmm.h — C ABI of the B200 (sm_100a) grouped-GEMM core library.
 *
 * Plain pointers and sizes only; no torch types cross this boundary.  All
 * functions return 0 on success or a negative B200GMM_E* code and never throw.
 * Work is enqueued on the CUDA stream the caller passes and is asynchronous
 * with respect to the host; no entry point synchronises the device unless its
 * comment says so.  Tensors are bf16, contiguous, row-major; batch_sizes is
 * int64.  The device current at the time of the call must own the pointers.
 *
 * Every declaration cites the piece of the reference (tgale96/grouped_gemm,
 * paths relative to that project) whose job it takes over.
 */
#ifndef B200GMM_H_
#define B200GMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error codes (b200gmm_strerror gives the text). */
#define B200GMM_OK 0
#define B200GMM_EINVAL -1       /* bad argument combination (e.g. both transposes) */
#define B200GMM_EALIGN -2       /* a row length is not a multiple of 8 elements */
#define B200GMM_ELIMIT -3       /* too many experts / too many tiles / dim too large */
#define B200GMM_EWORKSPACE -4   /* workspace missing, too small or misaligned */
#define B200GMM_ECUDA -5        /* a CUDA runtime or driver call failed */
#define B200GMM_ETENSORMAP -6   /* cuTensorMapEncodeTiled rejected a tensor */
#define B200GMM_EDEVICE -7      /* not an sm_100 device */
#define B200GMM_ETIMEOUT -8     /* (status word) a bounded wait inside the kernel gave up */

/* Largest number of experts one call accepts.  The reference caps the
 * device-side path at 512 (csrc/fill_arguments.cuh:11, csrc/grouped_gemm.cu:120-124). */
#define B200GMM_MAX_EXPERTS 1024

/* Bits of the device status word written by the kernels (0 = clean run). */
#define B200GMM_STATUS_TIMEOUT 0x1u        /* a bounded mbarrier wait ran out */
#define B200GMM_STATUS_NEGATIVE_SIZE 0x2u  /* a batch size was < 0 (treated as 0) */
#define B200GMM_STATUS_ROWS_OVERFLOW 0x4u  /* sum(batch_sizes) > rows of a (clamped) */
#define B200GMM_STATUS_BAD_ROW_INDEX 0x8u  /* run_gather: a row index outside x (read as zeros) */
#define B200GMM_STATUS_HANDOFF 0x20u       /* self-check: a role of a thread block was handed tile positions out of order */
#define B200GMM_STATUS_BAD_ROW_DEST 0x10u  /* a row_dest entry outside [dest_base, +dest_bytes) or not 16-byte aligned (row skipped) */

/* Largest number of experts b200gmm_run_static accepts (its built-in scratch is
 * sized for this many). */
#define B200GMM_STATIC_MAX_EXPERTS 256

/* Number of int64 fields b200gmm_fill_offsets writes per expert:
 * m, n, k, lda, ldb, ldc, a_offset, b_offset, c_offset (offsets in elements). */
#define B200GMM_FILL_FIELDS 9

/* Number of fields b200gmm_schedule_host / b200gmm_schedule_device write per tile:
 * expert, row0, col0, valid_rows, pipeline stages, kind (0: rows x 256 columns;
 * 1: transposed tile, all rows of an expert of at most 64 rows x 128 columns). */
#define B200GMM_SCHEDULE_FIELDS 6

/*
 * Bytes of device scratch b200gmm_run needs for `z` experts (about 0.5 MB).
 * The scratch holds a device copy of batch_sizes (when the caller's copy is in
 * host memory) and, for trans_a, per-CTA copies of the two TMA tensor maps whose
 * row extent the kernel clips at each expert's last row.  Two calls that may run
 * at the same time need separate workspaces.
 * Replaces the seven per-call torch::empty scratch tensors of
 * csrc/grouped_gemm.cu:119-138 (MakeArgumentsOnDevice) and the seven H2D copies
 * of csrc/grouped_gemm.cu:83-94, :209-218 (CopyToDevice).
 */
int b200gmm_workspace_bytes(int z, size_t* out_bytes);

/*
 * The grouped GEMM itself: one persistent kernel launch for all experts.
 * Two kernel variants exist (tiles owned by one CTA, or by a pair of CTAs on
 * neighbouring SMs); the choice depends only on the shapes passed here and can
 * be forced with the environment variable B200GMM_CTAS=1|2.  B200GMM_GROUP_M
 * overrides how many row-tiles are swept together across the columns.
 * Replaces grouped_gemm::GroupedGemm (csrc/grouped_gemm.cu:470-564, prototype
 * csrc/grouped_gemm.h:5-9) together with the argument fill
 * (csrc/fill_arguments.cuh:34-131) that precedes the CUTLASS launch.
 *
 *   trans_a=0, trans_b=0:  c[rows_i, :] = a[rows_i, :] @ b[i]        a[T,k] b[z,k,n] c[T,n]
 *   trans_a=0, trans_b=1:  c[rows_i, :] = a[rows_i, :] @ b[i]^T      a[T,k] b[z,n,k] c[T,n]
 *   trans_a=1, trans_b=0:  c[i] = a[rows_i, :]^T @ b[rows_i, :]      a[T,m] b[T,n]   c[z,m,n]
 *
 * rows_i is the i-th run of batch_sizes[i] consecutive rows.  `dim_a1` is
 * a's second dimension (k, or m when trans_a), `n` the output's last
 * dimension.  For trans_a every c[i] is written, as zeros when
 * batch_sizes[i]==0 (csrc/fill_arguments.cuh:100-119).  Rows of c past
 * sum(batch_sizes) are left untouched, as in the reference.
 *
 * batch_sizes may live in host memory (batch_sizes_on_device=0: it is copied
 * into the workspace with one cudaMemcpyAsync.  A pageable array is staged
 * before this call returns and may be reused at once; a PINNED array is read
 * later, when the stream reaches the copy, and must stay valid and unchanged
 * until then) or in device memory (=1: never read by the host, no
 * synchronisation).
 *
 * `workspace` is device memory of at least b200gmm_workspace_bytes(z) bytes,
 * 128-byte aligned, owned by the caller and reusable once the stream has passed
 * this call.  If `device_status` is non-NULL it must point to a 4-byte device
 * word that the kernel ORs B200GMM_STATUS_* bits into (the caller clears it).
 */
int b200gmm_run(const void* a, const void* b, void* c,
                const int64_t* batch_sizes, int batch_sizes_on_device,
                int z, int64_t tokens, int64_t dim_a1, int64_t n,
                int trans_a, int trans_b,
                void* workspace, size_t workspace_bytes,
                uint32_t* device_status, void* cuda_stream);

/*
 * b200gmm_run for callers that have no device memory to hand over and may not
 * create any: same arguments, same kernel and same results as b200gmm_run, but
 * without the workspace pair.  (This entry point has no counterpart in the
 * reference, which always allocates its scratch through torch.)
 *
 * Who needs it: code that runs where allocating is not an option -- an inference
 * server that has already given all free HBM to its own cache pool, a plugin
 * that is handed input and output buffers and nothing else, a latency-critical
 * thread that must not take the allocator's locks (after the first call on a
 * device this function takes no lock of its own either).  The scratch
 * (device copy of batch_sizes, per-CTA tensor-map copies) lives in a fixed
 * array inside the library image, about 0.5 MB, present on every GPU that loads
 * the library for as long as the process runs.  This function calls no
 * cudaMalloc / cudaFree and no allocating library routine.
 *
 * Limits and rules:
 *  - at most B200GMM_STATIC_MAX_EXPERTS experts; more returns B200GMM_ELIMIT
 *    and launches nothing;
 *  - the first call on each device looks up the array's device address (a few
 *    CUDA runtime queries with that device current); make that first call
 *    before starting any stream capture on that device;
 *  - all calls on one device share the one array.  Nothing in it has to start
 *    out zeroed (each call overwrites what it reads), but two calls whose
 *    kernels can overlap on the GPU -- different streams without an ordering
 *    between them -- race on it.  Keep such calls on one stream or order them
 *    with events; use b200gmm_run with separate workspaces for concurrency.
 */
int b200gmm_run_static(const void* a, const void* b, void* c,
                       const int64_t* batch_sizes, int batch_sizes_on_device,
                       int z, int64_t tokens, int64_t dim_a1, int64_t n,
                       int trans_a, int trans_b,
                       uint32_t* device_status, void* cuda_stream);

/*
 * b200gmm_run (trans_a = 0 only) with the expert-parallel combine fused into the
 * kernel's epilogue: row i of the result is not written to a c tensor but to the
 * address row_dest[i] (device array of `tokens` byte addresses, each 16-byte
 * aligned, each the start of an n-element bf16 row).  The addresses may point
 * into buffers on other GPUs that are mapped into this process (symmetric memory
 * or CUDA IPC): rows then leave over NVLink with plain stores while the tensor
 * cores work on the next tile, and no separate gather / all-to-all / scatter pass
 * over the output is needed.  Remote memory is only written.  The caller orders
 * the kernel against the readers on the other GPUs (a barrier after it).  Rows
 * past sum(batch_sizes) are not written.  Other arguments as in b200gmm_run.
 *
 * `dest_base` / `dest_bytes` declare the one buffer all destinations lie in: a
 * row whose address is below dest_base, whose n elements would end past
 * dest_base + dest_bytes, or whose address is not 16-byte aligned is NOT written
 * and B200GMM_STATUS_BAD_ROW_DEST is raised.  Pass the output tensor here
 * whenever the table was computed from indices of unknown provenance.  NULL / 0
 * switches the range check off for callers that built the table themselves, e.g.
 * from rows of several peer buffers; the alignment check always applies.  The same pair, with the same meaning, follows
 * row_dest in b200gmm_run_combine, b200gmm_run_gather and b200gmm_run_swiglu.
 * The reference has no counterpart (single GPU; its callers un-sort the output
 * themselves).
 */
int b200gmm_run_scatter(const void* a, const void* b, const int64_t* row_dest,
                        const void* dest_base, int64_t dest_bytes,
                        const int64_t* batch_sizes, int batch_sizes_on_device,
                        int z, int64_t tokens, int64_t dim_a1, int64_t n, int trans_b,
                        void* workspace, size_t workspace_bytes,
                        uint32_t* device_status, void* cuda_stream);

/*
 * b200gmm_run_scatter that also moves rows between GPUs while the product runs:
 * extra warps in every thread block (by default one thread of them, issuing bulk
 * async copies global -> shared -> destination; B200GMM_PUSH_TMA=0: four warps
 * copying through registers) carry out exactly the transfer
 * b200gmm_push_rows describes (push_* arguments as there: item i is row
 * push_src_row[i], or i when that is NULL, of push_src -> row push_dst_row[i] of
 * the buffer push_peer_base[push_dst_rank[i]]), so a dispatch that the NEXT
 * product needs - e.g. the gradient rows for dgrad, sent while the forward
 * product runs - costs no pass of its own and no second kernel shares the SMs.
 * The pushed rows are independent of the product; they are complete when the
 * launch is, and the caller orders them against their readers as after
 * b200gmm_push_rows.  No multicast; remote memory is only written.
 * If the product is empty the rows are moved by b200gmm_push_rows instead.
 * The reference has no counterpart (single GPU).
 */
int b200gmm_run_scatter_push(const void* a, const void* b, const int64_t* row_dest,
                             const void* dest_base, int64_t dest_bytes,
                             const int64_t* batch_sizes, int batch_sizes_on_device,
                             int z, int64_t tokens, int64_t dim_a1, int64_t n, int trans_b,
                             const void* push_src, int64_t push_row_bytes, int64_t push_items,
                             const int32_t* push_src_row, const int32_t* push_dst_rank,
                             const int64_t* push_dst_row, const void* const* push_peer_base,
                             void* workspace, size_t workspace_bytes,
                             uint32_t* device_status, void* cuda_stream);

/*
 * b200gmm_run_scatter with the router's weights and the top-k sum folded in:
 * row i of the product is multiplied by row_weight[i] (device float [tokens];
 * NULL = 1) in fp32 before it is rounded to bf16, and, if accumulate is
 * non-zero, ADDED to the bf16 row at row_dest[i] instead of overwriting it
 * (bulk reduce-add copies).  With top-k routing the k rows of one token, which
 * belong to k experts, carry the same destination: the caller zeroes the output,
 * one call sums all contributions.  The additions of different rows to one
 * destination happen in no defined order, each rounding to bf16, so results can
 * differ in the last bit from run to run.  Destinations in another GPU's memory
 * have been exercised with the plain copies of b200gmm_run_scatter only, not
 * with the reduce-add copies.  The reference has no counterpart: its callers
 * un-sort, weight and sum in kernels of their own.
 */
int b200gmm_run_combine(const void* a, const void* b, const int64_t* row_dest,
                        const void* dest_base, int64_t dest_bytes,
                        const float* row_weight, int accumulate,
                        const int64_t* batch_sizes, int batch_sizes_on_device, int z,
                        int64_t tokens, int64_t dim_a1, int64_t n, int trans_b,
                        void* workspace, size_t workspace_bytes,
                        uint32_t* device_status, void* cuda_stream);

/*
 * b200gmm_run (trans_a = 0 only) with the caller's sort-by-expert fused into the
 * operand load: row i of the grouped left operand is row row_index[i] of `x`
 * (bf16 [x_rows, dim_a1], contiguous; row_index: device int32 [tokens], values in
 * [0, x_rows)).  Extra warps of the kernel fetch those rows with 16-byte
 * cp.async copies into the swizzled tile layout the tensor core reads, so no
 * permuted copy of the activations is ever written.  An index outside
 * [0, x_rows) is not dereferenced: the row counts as zeros and
 * B200GMM_STATUS_BAD_ROW_INDEX is raised.  Cost on the Mixtral forward shape:
 * about 10 % more time than b200gmm_run on already permuted rows, on a par with
 * a separate gather followed by b200gmm_run.
 * Results go to c[i] as in b200gmm_run, or, if row_dest is non-NULL, to the
 * addresses row_dest[i] as in b200gmm_run_scatter (c may then be NULL).
 * The reference has no counterpart: its callers gather the rows into a new
 * tensor before calling gmm.
 */
int b200gmm_run_gather(const void* x, int64_t x_rows, const int32_t* row_index,
                       const void* b, void* c, const int64_t* row_dest,
                       const void* dest_base, int64_t dest_bytes,
                       const int64_t* batch_sizes, int batch_sizes_on_device,
                       int z, int64_t tokens, int64_t dim_a1, int64_t n, int trans_b,
                       void* workspace, size_t workspace_bytes,
                       uint32_t* device_status, void* cuda_stream);

/*
 * The weight gradient that goes with b200gmm_run_gather: for every expert i
 *   c[i] = x[row_index[rows_i], :]^T @ grad[rows_i, :]     ([dim_x1, n], zeros if empty)
 * i.e. b200gmm_run with trans_a = 1 whose left operand is gathered from `x`
 * (bf16 [x_rows, dim_x1]) through row_index (device int32 [tokens]) instead of
 * being read from a permuted copy.  grad is bf16 [tokens, n], grouped by expert;
 * c is bf16 [z, dim_x1, n].  Index checks as in b200gmm_run_gather.
 * (The input gradient of the gathered product is b200gmm_run_combine with
 * accumulate = 1 and the same row_index as destinations.)
 * The reference has no counterpart.
 */
int b200gmm_run_gather_wgrad(const void* x, int64_t x_rows, const int32_t* row_index,
                             const void* grad, void* c,
                             const int64_t* batch_sizes, int batch_sizes_on_device,
                             int z, int64_t tokens, int64_t dim_x1, int64_t n,
                             void* workspace, size_t workspace_bytes,
                             uint32_t* device_status, void* cuda_stream);

/*
 * Gated forward product of a SwiGLU expert layer in one kernel:
 *   c[rows_i, :] = silu(a[rows_i, :] @ b_gate[i]) * (a[rows_i, :] @ b_up[i])
 * with silu(x) = x / (1 + exp(-x)).  b_gate and b_up have the shape b has in
 * b200gmm_run with trans_a = 0 ([z, k, n], or [z, n, k] with trans_b); c is
 * bf16 [tokens, n].  Both products accumulate in fp32 in one 256-column
 * accumulator (128 gate columns, 128 up columns); the epilogue applies the gate
 * to the fp32 values and rounds once, so neither product is written to memory.
 * If row_dest is non-NULL the rows go to the addresses row_dest[i] as in
 * b200gmm_run_scatter (c may then be NULL).
 * The reference has no counterpart: its callers run gmm twice (or once on
 * concatenated weights) and apply the activation in a separate kernel.
 */
int b200gmm_run_swiglu(const void* a, const void* b_gate, const void* b_up, void* c,
                       const int64_t* row_dest, const void* dest_base, int64_t dest_bytes,
                       const int64_t* batch_sizes,
                       int batch_sizes_on_device, int z, int64_t tokens, int64_t dim_a1,
                       int64_t n, int trans_b, void* workspace, size_t workspace_bytes,
                       uint32_t* device_status, void* cuda_stream);

/*
 * Backward of b200gmm_run_swiglu with respect to its two products, in one
 * kernel: the gate and up products are recomputed in the accumulator (they were
 * never stored), and the epilogue reads grad_out (bf16 [tokens, n], the gradient
 * of c) and writes
 *   grad_products[0] = grad_out * up * silu'(gate)     silu'(g) = s (1 + g (1 - s)), s = 1 / (1 + exp(-g))
 *   grad_products[1] = grad_out * silu(gate)
 * into grad_products (bf16 [2, tokens, n], contiguous): the gradients of the
 * loss w.r.t. a @ b_gate and a @ b_up.  From them the caller gets the input
 * gradient with two b200gmm_run calls (trans_b flipped, summed) and the two
 * weight gradients with two trans_a calls, exactly as for a plain product
 * (grouped_gemm/ops.py:14-29 of the reference).  Rows past sum(batch_sizes) of
 * grad_products are left untouched.  The reference has no counterpart.
 */
int b200gmm_run_swiglu_backward(const void* a, const void* b_gate, const void* b_up,
                                const void* grad_out, void* grad_products,
                                const int64_t* batch_sizes, int batch_sizes_on_device,
                                int z, int64_t tokens, int64_t dim_a1, int64_t n, int trans_b,
                                void* workspace, size_t workspace_bytes,
                                uint32_t* device_status, void* cuda_stream);

/*
 * Row exchange for expert parallelism: copy `n_items` rows of `row_bytes` bytes
 * (a multiple of 16) from `src` on this GPU into rows of buffers that may live
 * on other GPUs.  Item i reads row src_row[i] of `src` (row i when src_row is
 * NULL) and writes row dst_row[i] of the buffer whose base address is
 * peer_base[dst_rank[i]].  All index arrays and the `peer_base` table are
 * device memory; the table holds addresses of peer buffers mapped into this
 * process (symmetric memory or CUDA IPC) and of this GPU's own buffer at its
 * own rank.  Plain loads and stores only: no TMA, no multicast, and remote
 * memory is only written, never read.  The caller orders the transfer against
 * the consumers on the other GPUs (a barrier after the push).  `max_ctas` > 0
 * caps the number of thread blocks (default: four per SM), for a transfer that
 * should leave memory bandwidth to other work.
 * The reference has no counterpart: it is single-GPU and leaves the
 * sort-by-expert permutation to its callers.
 */
int b200gmm_push_rows(const void* src, int64_t row_bytes, int64_t n_items,
                      const int32_t* src_row, const int32_t* dst_rank,
                      const int64_t* dst_row, const void* const* peer_base,
                      int max_ctas, void* cuda_stream);

/*
 * The top-k sum that ends an expert-parallel combine: `slots` is bf16
 * [tokens * top_k, cols] (the top_k result rows of a token are consecutive),
 * `out` is bf16 [tokens, cols]; out[t] = slots[t*top_k] + .. + slots[t*top_k +
 * top_k - 1], added in fp32 in that order, rounded once.  1 <= top_k <= 8, cols a
 * multiple of 8, both pointers 16-byte aligned device memory.  The reference has
 * no counterpart (its callers sum the expert outputs of a token themselves).
 */
int b200gmm_sum_slots(const void* slots, void* out, int64_t tokens, int top_k,
                      int64_t cols, void* cuda_stream);

/*
 * Device-side argument fill on its own, for inspection and bit-exact tests:
 * runs the same warp-scan step the GEMM kernels build their schedule from and
 * writes z x B200GMM_FILL_FIELDS int64 values (expert-major) to `out_device`.
 * Semantics of each field follow FillArguments (csrc/fill_arguments.cuh:59-78)
 * and its host twin MakeArgumentsOnHost (csrc/grouped_gemm.cu:160-175),
 * evaluated in int64.  `batch_sizes_device` must be device memory.
 */
int b200gmm_fill_offsets(const int64_t* batch_sizes_device, int z,
                         int64_t dim_a1, int64_t n, int trans_a, int trans_b,
                         int64_t* out_device, void* cuda_stream);

/*
 * Host replay of the tile schedule the persistent kernel walks (same
 * __host__ __device__ code as the kernel).  Writes, for every position of the
 * launch order, B200GMM_SCHEDULE_FIELDS int64 values into `out` (at most
 * `max_tiles` tiles) and the tile count into *n_tiles.  CTAs draw positions
 * from a global counter in this order; for trans_a, where a tile's duration
 * is its expert's row count, the experts are first sorted by their number of
 * rows, largest first (the reference sorts its wgrad problems the same way,
 * csrc/fill_arguments.cuh:80-86), so that the launch ends on short tiles.
 * `cluster_ctas` selects the kernel variant: 1 (each CTA owns 128-row tiles),
 * 2 (a pair of CTAs owns 256-row tiles) or 0 (whatever b200gmm_run would pick
 * for these shapes).  Pure host arithmetic; needs no GPU.  It has no
 * counterpart in the reference, whose schedule lives inside CUTLASS
 * (GroupScheduleMode::kDeviceOnly, csrc/grouped_gemm.cu:256-259).
 */
int b200gmm_schedule_host(const int64_t* batch_sizes_host, int z,
                          int64_t tokens, int64_t dim_a1, int64_t n,
                          int trans_a, int trans_b, int cluster_ctas,
                          int64_t* out, int64_t max_tiles, int64_t* n_tiles);

/*
 * The same schedule as the GPU builds it: one CTA runs the GEMM kernels' own
 * prologue (prefix sums of batch_sizes, expert order, tile prefix sums) and
 * tile decoder and writes B200GMM_SCHEDULE_FIELDS int32 values per tile into
 * `out_device` (at most `max_tiles` tiles) and the tile count into
 * *n_tiles_device.  For tests: the result must equal b200gmm_schedule_host's
 * exactly.  Replaces nothing in the reference (its tests never look at the
 * argument arrays FillArguments writes, csrc/fill_arguments.cuh:88-97).
 */
int b200gmm_schedule_device(const int64_t* batch_sizes_device, int z,
                            int64_t tokens, int64_t dim_a1, int64_t n,
                            int trans_a, int trans_b, int cluster_ctas,
                            int32_t* out_device, int64_t max_tiles,
                            int32_t* n_tiles_device, uint32_t* device_status,
                            void* cuda_stream);

/*
 * Exercises the kernels' bounded wait in isolation: one warp waits on an
 * mbarrier that nothing signals, gives up after `limit_ns` nanoseconds (at most
 * 100 ms) and ORs B200GMM_STATUS_TIMEOUT into *device_status, which is how every
 * wait inside the GEMM kernels ends if its partner never arrives (their limit is
 * 2 s, or B200GMM_WAIT_LIMIT_NS nanoseconds from the environment).  No copy or
 * MMA is in flight, nothing faults, the context stays usable.  The reference has
 * no counterpart (its kernels have no waits of their own).
 */
int b200gmm_selftest_wait_timeout(int64_t limit_ns, uint32_t* device_status,
                                  void* cuda_stream);

/* Tile shape of a kernel variant (cluster_ctas = 1 or 2): out[0]=rows,
 * out[1]=cols, out[2]=k depth per pipeline stage. */
int b200gmm_tile_shape(int cluster_ctas, int* out3);

/* Number of kernels this library has launched in this process (all entry
 * points), for launch accounting in benchmarks. */
int64_t b200gmm_launch_count(void);

/* Text for an error code.  Replaces the TORCH_CHECK messages of
 * csrc/grouped_gemm.cu:21-32. */
const char* b200gmm_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* B200GMM_H_ */
