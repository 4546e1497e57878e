/*
 * b200_sgemm — C ABI of the B200 (sm_100a) FP32 GEMM library.
 *
 * This is the boundary a binding of the reference's operator would call: plain pointers, sizes and
 * integers only.  Matrices are FP32 in device memory; layouts are 0 = row-major, 1 = col-major
 * (the enumerator order of rocm_sgemm::m_layout, rocm_sgemm/include/rocm_sgemm/kernel/common.hpp:36-40).
 * Every function returns a status (0 = OK) instead of throwing or exiting; the C++ shim
 * include/rocm_sgemm/gemm.hpp turns a non-zero status into std::runtime_error, the one throwing
 * behaviour the reference has (rocm_sgemm/include/rocm_sgemm/kernel_launcher.hpp:89-94).
 * There is no CPU fallback: without a CUDA device the compute entry points return a CUDA error.
 */
#ifndef B200_SGEMM_H
#define B200_SGEMM_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_SGEMM_ROW_MAJOR 0
#define B200_SGEMM_COL_MAJOR 1

/* status codes; positive values are cudaError_t codes reported by the CUDA runtime */
#define B200_SGEMM_OK 0
#define B200_SGEMM_INVALID_ARGUMENT (-1) /* null pointer, zero dimension, bad layout, bad leading dimension */
#define B200_SGEMM_NO_KERNEL (-2)        /* no kernel built for (variant, layout, alignment) */
#define B200_SGEMM_WORKSPACE_TOO_SMALL (-3)
#define B200_SGEMM_UNSUPPORTED_SIZE (-4) /* a dimension exceeds what the kernels index (2^31-1) */
#define B200_SGEMM_SCRATCH_LIMIT (-5)    /* b200_sgemm_splitk_static: split_k * M * N floats exceed the built-in scratch */

/* Tile parameters of one kernel variant: the reference's nine (struct gemm_params emitted by
 * rocm_sgemm/config/generate_config.py:100-111) followed by the CUDA-side additions. */
typedef struct b200_sgemm_params
{
    int block_size;        /* threads per CTA */
    int block_m;           /* CTA tile rows */
    int block_n;           /* CTA tile columns */
    int block_k;           /* K depth of one staged tile */
    int warp_tile_m_count; /* thread sub-tiles per thread along m */
    int warp_tile_n_count; /* thread sub-tiles per thread along n */
    int thread_tile_m;     /* rows of one thread sub-tile (one shared-memory vector read) */
    int thread_tile_n;     /* columns of one thread sub-tile */
    int threads_n;         /* lanes of a warp along n */
    int stages;            /* depth of the shared-memory ring */
    int fma_mode;          /* 0 scalar fma.rn.f32, 1 fma.rn.f32x2 (A duplicated), 2 fma.rn.f32x2 (2x2 diagonal) */
    int raster;            /* 0 row-major tile order, 1 grouped bands, 2 Hilbert curve */
    int min_blocks;        /* CTAs per SM the register budget is sized for */
    int pipeline;          /* 0 every warp stages and computes, 1 warp-specialised (TMA / producer warps + mbarriers) */
    int split_k;           /* K slices chosen for the looked-up problem (1 = none) */
    int pretranspose;      /* bit 0 / 1: b200_sgemm multiplies a K-contiguous A / B from an M / N-contiguous copy in scratch */
} b200_sgemm_params;

/* C = A*B, C overwritten, packed matrices, asynchronous on `cuda_stream` (a cudaStream_t; NULL = the
 * default stream), no synchronisation and no error check of the kernel's execution.
 * Replaces rocm_sgemm::gemm<layout_C, layout_A, layout_B>(C, A, B, M, N, K, stream)
 * (rocm_sgemm/include/rocm_sgemm/gemm.hpp:51-52, rocm_sgemm/src/gemm.cpp:8-41): same argument order
 * (C, A, B), same semantics (alpha = 1, beta = 0, inputs untouched), additionally correct for ragged
 * M, N, K.  A is MxK, B is KxN, C is MxN.  Scratch comes from an internal per-(device, stream) arena that
 * grows on demand: the accumulator parking slots of the balanced schedules (one CTA tile per SM, whenever the
 * tiles do not fill the last wave), split-K partial sums where the tuned table still slices K, and, where the
 * table entry asks for it and the problem is large enough for it to pay (the other dimension >= 1024), the
 * transposed copy of a K-contiguous operand (row-major A, col-major B), so that the hot kernel can fetch it
 * straight with TMA.  The warp-specialised kernels make that copy themselves, block by block ahead of their own
 * reads (each block once for all CTAs, by producer warps that would otherwise idle); a transposition kernel in
 * front of the product makes it where that does not apply.  About 0.8 % extra time per operand at 4096^3, instead
 * of 3.5 % for transposing every tile where it is consumed.  b200_sgemm_ex never copies an operand: it runs
 * exactly the kernel it is told.
 * Not for stream capture: the flag words behind the balanced schedules and the in-kernel transposition carry a
 * number that the host advances with every call, which a replayed graph would repeat.  (b200_sgemm_ex without a
 * workspace runs the plain schedule, uses no flag words and can be captured.) */
int b200_sgemm(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B, size_t M, size_t N,
               size_t K, void* cuda_stream);

/* Same operation with everything the drop-in entry decides made explicit: leading dimensions in
 * elements (0 = packed), a forced kernel variant (-1 = look up the table, as
 * detail::find_best_config does in rocm_sgemm/src/gemm.cpp:12), a forced split-K (0 = the table's when the
 * variant is looked up, no split with a forced variant; n >= 2 = n equal K slices summed in order by a second
 * kernel; -1 = equal K ranges per CTA summed in order inside the kernel, for problems with fewer tiles than SMs)
 * and a caller-owned workspace (required for n >= 2 slices: at least b200_sgemm_workspace_bytes(); optional
 * otherwise, see there).  The tuner drives kernels through this
 * entry the way the reference's tuner launches a JIT-compiled instantiation directly
 * (rocm_sgemm/config/tuner.cpp:419-429); the column-sharded multi-GPU driver uses the leading
 * dimensions. */
int b200_sgemm_ex(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B, size_t M,
                  size_t N, size_t K, size_t lda, size_t ldb, size_t ldc, int variant, int split_k, void* workspace,
                  size_t workspace_bytes, void* cuda_stream);

/* One tuning trial: exactly what b200_sgemm does for a problem whose table entry names this kernel variant,
 * split_k (1 = none, n >= 2 = n slices + reduction kernel, 0 = equal K ranges per CTA) and pretranspose bits
 * (bit 0 / 1: a K-contiguous A / B is multiplied from a transposed copy in the arena; the warp-specialised
 * kernels make that copy themselves, block by block ahead of their own reads, and bit 2 of a trial asks for a
 * transposition kernel in front of the product instead, which is also what the other kernels get) - scratch from
 * the library's arena, the balanced schedules where they apply.  The tuner times candidates through this entry, so that every property of
 * a table entry is searched through the path the drop-in entry takes; the reference's tuner launches its
 * JIT-compiled instantiation directly (rocm_sgemm/config/tuner.cpp:419-429). */
int b200_sgemm_trial(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B, size_t M,
                     size_t N, size_t K, int variant, int split_k, int pretranspose, void* cuda_stream);

/* The product written to several destinations at once: C_list[0 .. n_dst-1] (1 <= n_dst <= 8) all receive the
 * M x N result with the same layout and leading dimension; the kernel's epilogue stores every tile to each of them.
 * Meant for the column-sharded multi-GPU product: each GPU passes the position of its own column block inside its
 * own C and inside every peer's C (peer mappings obtained with CUDA IPC or any other peer-access mechanism), so that
 * when all GPUs have finished every GPU holds the whole C and the all-gather that would follow
 * (the reference has no multi-GPU path; its matrices live on one device, test/gemm/test.cpp:50-74) is
 * folded into the GEMM.  Plain stores only; the caller synchronises the GPUs before reading C.  Runs the
 * warp-specialised kernels without split-K: B200_SGEMM_NO_KERNEL if `variant` (-1 = the table's) is another kind.
 * With variant = -1 the table entry may, as in b200_sgemm, pre-transpose a K-contiguous operand into the
 * library's per-(device, stream) arena. */
int b200_sgemm_multi(int layout_c, int layout_a, int layout_b, float* const* C_list, int n_dst, const float* A,
                     const float* B, size_t M, size_t N, size_t K, size_t lda, size_t ldb, size_t ldc, int variant,
                     void* cuda_stream);

/* The K cut points of the "equal ranges" schedule (split_k -1 in b200_sgemm_ex, split_k 0 in a table entry) for
 * a problem on a device with sm_count SMs, so that a host-side check can restate the arithmetic: every tile's K
 * extent is cut at the reported points, each piece is a k-ascending FMA chain from zero, and C is the last piece's
 * chain plus the earlier pieces, added one by one in ascending K order: ((p_last + p_0) + p_1) + ...  Tiles are block_mnk[0] x block_mnk[1] (block_mnk[2] = the K tile), numbered
 * tile_row * ceil(N / block_n) + tile_column; offsets[t] .. offsets[t+1] index tile t's cut points in `bounds` (K
 * positions strictly between 0 and K).  Returns the total number of cut points (0 = this call would not use the
 * schedule: no cuts at all, or equal slices), negative = error; at most `capacity` entries of either array are
 * written (offsets needs tiles + 1).  No reference counterpart: the reference's kernel never splits K. */
int b200_sgemm_stream_plan(int layout_c, int layout_a, int layout_b, size_t M, size_t N, size_t K, int variant,
                           int split_k, int sm_count, int* block_mnk, int* offsets, int* bounds, int capacity);

/* Bytes of workspace b200_sgemm_ex can use for this call: the split-K partial sums when the effective split is
 * > 1 (required), else the accumulator parking slots of the balanced schedules on the current device (optional:
 * with a smaller or no workspace the call runs the plain schedule and, unless split_k is -1, computes the same
 * bits), else 0. */
size_t b200_sgemm_workspace_bytes(int layout_c, int layout_a, int layout_b, size_t M, size_t N, size_t K, int variant,
                                  int split_k);

/* Table lookup without launching: fills `out` (may be NULL) and `variant` (may be NULL).
 * Replaces rocm_sgemm::get_gemm_params(m, n, k, layout_c, layout_a, layout_b)
 * (rocm_sgemm/config/generate_config.py:282-303) and detail::find_best_config (:241-267). */
int b200_sgemm_select_config(int layout_c, int layout_a, int layout_b, size_t M, size_t N, size_t K,
                             b200_sgemm_params* out, int* variant);

/* Number of kernel variants (the reference's KERNEL_VARIANTS, generate_config.py:97) and their
 * parameters (detail::kernel_configs, :113-124). */
int b200_sgemm_num_variants(void);
int b200_sgemm_get_variant(int variant, b200_sgemm_params* out);

/* The tuned table itself (detail::sorted_config_map, generate_config.py:156-171):
 * mnk = {M, N, K}; layouts = {A, B, C}. */
int b200_sgemm_num_entries(void);
int b200_sgemm_get_entry(int index, size_t mnk[3], int layouts[3], int* variant, int* split_k);
int b200_sgemm_get_entry_pretranspose(int index); /* the entry's pretranspose bits, or -1 */

/* 1 when a kernel exists for (variant, layout index A*4+B*2+C, aligned 0/1), as a non-null
 * kernel_table slot does in the reference (rocm_sgemm/include/rocm_sgemm/kernel_lookup.hpp:39). */
int b200_sgemm_has_kernel(int variant, int layout_index, int aligned);

/* Tile order of a kernel variant's `raster` mode: position `id` (0 <= id < grid_m * grid_n) in the order
 * the CTAs walk the tile grid -> tile coordinates.  0 row-major, 1 bands of eight tile rows, 2 Hilbert
 * curve.  Host-side evaluation of the kernels' own mapping function (the reference's tile_mapper,
 * rocm_sgemm/include/rocm_sgemm/kernel/mapping.hpp:211-237, is device-only). */
int b200_sgemm_map_tile(int raster, int id, int grid_m, int grid_n, int* tile_m, int* tile_n);

/* The selection rule applied to a caller-supplied table (host only, no CUDA): `keys` holds `count`
 * rows of {m, n, k, layout_a, layout_b, layout_c} sorted the way the reference sorts them.
 * Returns the chosen row or -1 for an empty table. */
int b200_sgemm_select_in_table(const size_t* keys, size_t count, size_t M, size_t N, size_t K, int layout_a,
                               int layout_b, int layout_c);

/* Register-only FP32 FMA throughput probe on the current device: the measured FMA-pipe ceiling the
 * GEMM numbers are quoted against.  mode 0 = fma.rn.f32, 1 = fma.rn.f32x2.  Writes the elapsed
 * milliseconds of one launch (CUDA events on `cuda_stream`) and the FLOPs it performed. */
int b200_sgemm_fma_peak(int mode, int iterations, float* elapsed_ms, double* flops, void* cuda_stream);

/* Reads (and clears) the current device's kernel status word after synchronising the device:
 * 0 = no kernel reported a problem; 1 / 2 = a warp-specialised kernel gave up a bounded wait on a
 * shared-memory barrier (consumer / producer side), 3 = on another CTA's parked accumulators, 4 = on a block of
 * an operand that the kernel transposes itself; its output is then invalid.  Diagnostic only: the
 * reference has no counterpart because its kernel has no waits that could time out. */
int b200_sgemm_device_status(int* status);

/* Self-test of the kernels' bounded waits, safe to run on any device: launches a private copy of the
 * warp-specialised kernel whose wait limit is one millisecond on a single 128 x 128 x 64 tile (A: 128 x 64 col-major,
 * B: 64 x 128 row-major, C: 128 x 128 row-major device buffers, A and B 16-byte aligned) and withholds the second K
 * tile from it.  The consumer warps give up after the limit, record status 1 and return; C is left untouched.
 * Afterwards b200_sgemm_device_status() reads 1 once and 0 from then on.  Nothing traps and nothing stays in flight. */
int b200_sgemm_selftest_bounded_wait(float* C, const float* A, const float* B, void* cuda_stream);

/* The same operation for matrices in HOST memory: uploads row panels of A and column panels of B
 * alternately, computes the rectangle of C that each upload completes as one GEMM, downloads it when it
 * is done (upload, compute and download overlap on internal streams), and returns when C is
 * complete in host memory.  This is the sequence the reference's harness performs step by step
 * (test/gemm/test.cpp:50-74: hipMemcpy H2D, gemm, hipMemcpy D2H) folded into one call; page-locked host
 * buffers are needed for the overlap.  Device buffers come from a per-device arena of the library
 * (b200_sgemm_shutdown_host releases it).
 * b200_sgemm_host_submit only enqueues the job on the current device and returns a ticket; b200_sgemm_host_wait
 * (same device current) blocks until that job's C is complete in host memory; the host buffers must stay valid and
 * untouched in between.  Two jobs may be in flight per device (a third submit first waits for the oldest): the
 * uploads of the next job then overlap the compute-bound tail and the downloads of the current one, so a stream
 * of jobs runs at the pace of the uploads.  b200_sgemm_host = submit + wait. */
int b200_sgemm_host(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B, size_t M,
                    size_t N, size_t K);
int b200_sgemm_host_submit(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B, size_t M,
                           size_t N, size_t K, long long* ticket);
int b200_sgemm_host_wait(long long ticket);
/* The schedule the host-buffer entries use for an M x N x K problem on a device with sm_count SMs, without touching a
 * device: returns the number of strips of C (one GEMM each, in launch order) and writes the first `capacity` of them
 * as (first row, rows, first column, columns) into rects[4*i..] and their split-K factors into splits[i].  The
 * strips tile C exactly once.  Negative return = B200_SGEMM_INVALID_ARGUMENT.
 * b200_sgemm_host_plan is the schedule of a job that finds the pipeline empty (pieces of about 512 rows / columns:
 * the first strip starts after a few megabytes, for the latency of a single call); _pipelined the one of a job
 * submitted while another is still in flight (pieces of about 2048: every strip then has at least 148 tiles and runs
 * at the full kernel's rate, so that a stream of jobs goes at the pace of the uploads). */
int b200_sgemm_host_plan(size_t M, size_t N, size_t K, int sm_count, size_t* rects, int* splits, int capacity);
int b200_sgemm_host_plan_pipelined(size_t M, size_t N, size_t K, int sm_count, size_t* rects, int* splits, int capacity);
int b200_sgemm_shutdown_host(void);

/* The same product for `batch` matrices at fixed element strides: matrix b uses C + b*stride_c, A + b*stride_a,
 * B + b*stride_b (stride_a or stride_b may be 0 to share an operand; the C matrices must not overlap).  The
 * reference's benchmark has a --batch_count switch that only replicates buffers
 * (benchmark/gemm/bench.cpp:49-64,213-216); this entry computes every matrix, with the drop-in entry's table
 * lookup and arena.  A batch (batch > 1) is ONE launch of a warp-specialised kernel: the persistent CTAs walk the
 * tiles of all matrices (the batch is one more dimension of the tensor maps), so a batch of small problems fills the
 * SMs.  The matrices are the parallel work, so a batch never slices K, whatever the table entry of the single
 * problem says (an entry with K slices or a kernel of the other pipeline is replaced by a warp-specialised variant
 * built for the layout): every matrix is one k-ascending FMA chain per element.  K-contiguous operands go through
 * the kernel's staging ring and strides that are not multiples of 4 floats through its guarded route.  Only when
 * no such kernel is built for the layout: one launch per matrix on the stream, each as b200_sgemm would run it. */
int b200_sgemm_strided_batched(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                               size_t M, size_t N, size_t K, size_t stride_c, size_t stride_a, size_t stride_b,
                               size_t batch, void* cuda_stream);

/* Vendor-BLAS calling convention on this library's kernels: column-major C (ldc >= M),
 * C = alpha * op(A) * op(B) + beta * C, op(X) = X or X^T by trans_x (0 / 1), A stored (trans_a ? K x M : M x K)
 * with lda, B stored (trans_b ? N x K : K x N) with ldb.  With alpha = 1 and beta = 0 this is the mapping of
 * rocblas_wrapper::gemm<TRANSPOSE_A, TRANSPOSE_B> (rocblas_wrapper/src/gemm.cpp:45-60) and takes the path of
 * b200_sgemm (table entry, arena scratch, transposed copies, balanced schedules) with leading dimensions.
 * Otherwise every element is fl(fl(alpha*t) + fl(beta*c)) (three FP32 roundings, no contraction; beta = 0 does not
 * read C), formed in the epilogue of the warp-specialised kernels: no extra pass (measured at 4096^3: alpha = 2,
 * beta = 0 costs nothing, beta = 0.5 adds the read of C, 1 %).  Only where the table's kernel slices K or is of
 * the other pipeline the product goes to a per-(device, stream) scratch matrix and one more pass forms C;
 * b200_sgemm_blas_shutdown frees that scratch. */
int b200_sgemm_blas(int trans_a, int trans_b, size_t M, size_t N, size_t K, float alpha, const float* A, size_t lda,
                    const float* B, size_t ldb, float beta, float* C, size_t ldc, void* cuda_stream);
int b200_sgemm_blas_shutdown(void);

/* Optional comparison column, NOT part of the reference's surface and NOT its arithmetic: the same
 * C = A * B computed on the tensor cores (tcgen05, accumulators in tensor memory) with every FP32 operand
 * split into two TF32 halves and three products per pair ("3xTF32").  The result differs from the FP32 FMA
 * chain of b200_sgemm in the last few bits (relative error of about 2e-6 against float64; identity B does not
 * reproduce A bit for bit).  Same arguments as b200_sgemm.  Operands that are not K-contiguous (col-major A,
 * row-major B) or whose rows are not 16-byte aligned are first repacked into scratch kept per (device, stream)
 * (first such call on a stream allocates; b200_sgemm_3xtf32_shutdown frees it).  b200_sgemm_3xtf32_device_status
 * synchronises the device and returns (and clears) the kernel's status word: 0 unless a bounded wait
 * inside the kernel gave up. */
int b200_sgemm_3xtf32(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B, size_t M,
                      size_t N, size_t K, void* cuda_stream);
int b200_sgemm_3xtf32_device_status(void);
int b200_sgemm_3xtf32_shutdown(void);

/* Size of the scratch array that b200_sgemm_splitk_static uses; it is part of the library's device image. */
#define B200_SGEMM_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

/* Split-K GEMM for callers that cannot allocate device memory and cannot pass a workspace: hosts whose
 * memory pool already owns the whole device, latency-bound threads that must stay out of the driver's
 * allocator, plug-ins barred from allocating after their init hook.  Same operation and arguments as
 * b200_sgemm plus the number of K slices (>= 2); the partial sums live in a fixed
 * B200_SGEMM_STATIC_SCRATCH_BYTES array inside the library's device image, which every GPU the entry point
 * was called on holds until the process exits.  The call itself calls no allocation routine.  split_k * M * N * 4
 * bytes must fit the array, else B200_SGEMM_SCRATCH_LIMIT is returned and nothing runs.  The first call on a
 * device resolves the array's device address, and with CUDA's default lazy module loading that is also the
 * moment the driver loads the module and reserves the array (free device memory drops by about the array's size
 * during that one call; later calls leave it unchanged): make that first call in the host's initialisation phase,
 * before any stream capture on the device, or run with CUDA_MODULE_LOADING=EAGER.  All
 * calls share the array (it keeps the previous call's contents; no part of it needs clearing because
 * every slice is fully written before it is read), so calls that can overlap on the GPU race: keep them
 * on one stream or order them with events.
 * This entry point has no counterpart in the reference, whose kernel needs no scratch memory. */
int b200_sgemm_splitk_static(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                             size_t M, size_t N, size_t K, int split_k, void* cuda_stream);

/* Frees the scratch arena that b200_sgemm keeps for (current device, this stream), after waiting for the work queued
 * on the stream.  The arenas are keyed on the stream handle: call this before destroying a stream that the drop-in
 * entry has been used on, otherwise its arena stays allocated until b200_sgemm_shutdown (and a later stream that gets
 * the same handle value inherits it, which is harmless).  Unknown streams are not an error. */
int b200_sgemm_release_stream(void* cuda_stream);

/* Frees the internal split-K arenas of every device (optional; they are also freed at unload). */
int b200_sgemm_shutdown(void);

/* Human-readable text for a status returned by any function above. */
const char* b200_sgemm_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif /* B200_SGEMM_H */
