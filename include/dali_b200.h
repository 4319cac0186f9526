/* dali_b200 -- C ABI of the B200 (sm_100a) back end for Dali's lazy
 * expression -> optimize -> compile -> cache -> run path.
 *
 * The reference has no foreign-function interface; the seam this library
 * replaces is the one between the expression graph and the code it used to
 * generate:
 *   - the compiled-module entry point
 *       extern "C" void maker(void** array_data, const int* offsets,
 *                             const int** sizes, const int** strides,
 *                             const void** scalar_arguments, const int** shapes)
 *     (dali/utils/compiler.cpp:181-200, argument list dali/array/jit/jit.cpp:1030-1038),
 *   - the compile-or-load step Compiler::load / Compiler::compile keyed by a
 *     64-bit hash (dali/utils/compiler.h:91-173, dali/array/jit/jit.cpp:1011-1039),
 *   - the GEMM implementation registered for op::MatMul
 *     (dali/array/gemm/cublas_gemm.cu:110-198).
 *
 * Everything here is plain C: pointers, sizes, integer status codes.  Every
 * function returns DALIB200_OK (0) or a negative status; the message of the
 * last failure on the calling thread is read with dalib200_last_error().
 * There is no CPU fallback: without a CUDA device every compute entry point
 * fails with DALIB200_ERR_NO_DEVICE.
 */
#ifndef DALI_B200_H
#define DALI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DALIB200_ABI_VERSION 1

enum dalib200_status {
    DALIB200_OK = 0,
    DALIB200_ERR_INVALID = -1,     /* bad argument / malformed IR / shape mismatch */
    DALIB200_ERR_NO_DEVICE = -2,   /* no CUDA device or driver */
    DALIB200_ERR_COMPILE = -3,     /* NVRTC rejected the generated kernel (log in last_error) */
    DALIB200_ERR_CUDA = -4,        /* a CUDA runtime/driver call failed */
    DALIB200_ERR_NOT_FOUND = -5,   /* unknown kernel hash */
    DALIB200_ERR_UNSUPPORTED = -6, /* valid request the back end has no kernel for */
    DALIB200_ERR_TOO_LARGE = -7    /* size beyond a documented fixed limit */
};

/* element types.  0..2 are the reference's DType values
 * (dali/array/dtype.h:6-10); bf16 is a storage type: kernel arguments and GEMM
 * operands may be bf16, loads widen to fp32 exactly and stores round to nearest even. */
enum dalib200_dtype {
    DALIB200_F32 = 0,
    DALIB200_F64 = 1,
    DALIB200_I32 = 2,
    DALIB200_BF16 = 3
};

/* Copies the calling thread's last error message (NUL-terminated, truncated
 * to `capacity`) into `buffer`; returns the full length. */
size_t dalib200_last_error(char* buffer, size_t capacity);

/* Library / ABI version (DALIB200_ABI_VERSION). */
int dalib200_abi_version(void);

/* Binds the library to the first `n_gpus` visible CUDA devices (n_gpus <= 0:
 * all of them), creates their primary contexts and per-device scratch
 * arenas.  Idempotent.  Replaces the reference's implicit device set-up in
 * memory::allocate (dali/array/memory/memory_ops.cu.cpp:59-75). */
int dalib200_init(int n_gpus);

/* Number of devices bound by dalib200_init (0 before it / without a GPU). */
int dalib200_device_count(void);

/* ---- compile cache -------------------------------------------------------
 * Replaces Compiler::load / is_loaded / compile
 * (dali/utils/compiler.h:91-173, dali/utils/compiler.cpp:68-227).           */

/* Registers the fused-expression program `ir` (text, see dali_b200/csrc/ir.h)
 * under the caller's structural hash (the reference's kernel key,
 * dali/array/jit/jit.cpp:1017-1021).  Parses and validates it; kernels are
 * generated per concrete layout on first launch (or by dalib200_precompile)
 * and kept in memory and on disk.  Registering the same hash again with the
 * same text is a no-op; with different text it fails (hash collision). */
int dalib200_compile(uint64_t hash, const char* ir, size_t ir_len);

/* 1 if `hash` is registered in this process, else 0. */
int dalib200_is_loaded(uint64_t hash);

/* Generates and NVRTC-compiles (sm_100a) the kernel of `hash` for the layout
 * described exactly as in dalib200_launch, without launching.  Works without
 * a GPU.  On success *cubin_size (if non-NULL) receives the image size. */
int dalib200_precompile(uint64_t hash,
                        const int64_t* space, int space_rank,
                        void* const* array_data, const int64_t* offsets,
                        const int64_t* const* strides, int n_arrays,
                        size_t* cubin_size);

/* Directory of the on-disk cache (<dir>/<key>.cubin, .cu, .log).  Default:
 * $DALI_CACHE_DIR, else ~/.dali_b200/cache/ (reference default ~/.dali/cache/,
 * dali/utils/compiler.cpp:234-238).  Setting DALI_JIT_ALWAYS_RECOMPILE=true
 * ignores cached images once per process, as dali/array/jit/jit.cpp:27-47. */
int dalib200_cache_set_dir(const char* dir);
size_t dalib200_cache_get_dir(char* buffer, size_t capacity);
/* Drops every in-memory module (and with remove_files != 0 the files too). */
int dalib200_cache_clear(int remove_files);
/* Counters: [0] programs registered, [1] kernels in memory, [2] NVRTC
 * compilations, [3] disk hits, [4] launches. */
int dalib200_cache_stats(uint64_t stats[5]);

/* ---- launch ----------------------------------------------------------------
 * Replaces the call `compiled_self(data_ptrs, offsets, shapes, strides,
 * scalars, shapes_for_nodes)` (dali/array/jit/jit.cpp:1216-1223).
 *
 *  device      index among the devices bound by dalib200_init
 *  stream      a cudaStream_t / CUstream (NULL = the legacy default stream)
 *  space       extents of the program's iteration space, outermost first;
 *              space_rank must equal the rank the program declares
 *  array_data  DEVICE base pointer of the i-th distinct buffer, in the order
 *              the program declares its args (first-visit order, as
 *              SymbolTable::declare_array, dali/array/jit/jit.cpp:75-87)
 *  offsets     element offset of each view into its buffer
 *  strides     per arg, `space_rank` element strides of the view expressed in
 *              iteration-space coordinates (0 = broadcast along that dim);
 *              a NULL entry means "contiguous over the whole space"
 *  scalars     pointer to each scalar argument's value in HOST memory, read
 *              at launch (as ScalarView, dali/array/jit/scalar_view.cpp:44)
 * The call is asynchronous on `stream`; it never allocates caller-visible
 * memory and never frees caller memory. */
int dalib200_launch(uint64_t hash, int device, void* stream,
                    const int64_t* space, int space_rank,
                    void* const* array_data, const int64_t* offsets,
                    const int64_t* const* strides, int n_arrays,
                    const void* const* scalars, int n_scalars);

/* Same computation with HOST arrays: copies every read arg to the device,
 * launches, copies every written arg back and synchronises.  `extents[i]` is
 * the number of elements of buffer i.  This is the path a caller holding
 * host memory pays for (the reference pays it inside
 * SynchronizedMemory::move_to, dali/array/memory/synchronized_memory.cpp:237-269). */
int dalib200_launch_host(uint64_t hash, int device,
                         const int64_t* space, int space_rank,
                         void* const* host_data, const int64_t* extents,
                         const int64_t* offsets,
                         const int64_t* const* strides, int n_arrays,
                         const void* const* scalars, int n_scalars);

/* Name of the kernel skeleton ("map", "row", "col", "all") and launch
 * geometry the last dalib200_launch / _precompile on this thread selected;
 * for tests and profiles. */
size_t dalib200_last_variant(char* buffer, size_t capacity);

/* ---- GEMM -------------------------------------------------------------------
 * C[m,n] = alpha * A[m,k] . B[k,n] + beta * C, every operand addressed by
 * element strides (row stride, column stride), so contiguous, transposed and
 * strided views all pass as they are.  dtype: DALIB200_F32 / F64 / I32 (I32
 * accumulates in int32 like the reference's ReferenceGemm<int>).  Replaces
 * CublasGemmImpl::run (dali/array/gemm/cublas_gemm.cu:110-186), whose beta is
 * hard-wired to 0, and CpuGemmImpl::run (dali/array/gemm/cpu_gemm.cpp:22-84).
 * Asynchronous on `stream`. */
int dalib200_gemm(int device, void* stream, int dtype,
                  int64_t m, int64_t n, int64_t k,
                  const void* a, int64_t a_row_stride, int64_t a_col_stride,
                  const void* b, int64_t b_row_stride, int64_t b_col_stride,
                  void* c, int64_t c_row_stride, int64_t c_col_stride,
                  double alpha, double beta);

/* Tensor-core GEMM (tcgen05.mma, accumulator in tensor memory, operand tiles
 * staged by TMA) with the elementwise expression that consumes the product
 * spliced in as its epilogue, so the product never goes to memory on its own:
 *
 *     acc[m,n] = A[m,k] . B[k,n]          fp32 accumulation
 *     epilogue(acc, extra operands) -> destination(s)
 *
 * A and B are row-major with row pitches lda / ldb (elements), 16-byte aligned.
 *   ab_dtype DALIB200_BF16: one bf16 pass.
 *   ab_dtype DALIB200_F32 : three TF32 passes on operands split into a high
 *     and a low part (fp32 parity with an fp32 GEMM).  With a_lo = b_lo = NULL the
 *     parts are made in pool temporaries (recycled in stream order; k and n must
 *     be multiples of 4).  To reuse them across calls (weights), pass the parts
 *     made by dalib200_gemm_split_tf32: a / a_lo = parts of A, [m,k] with pitch lda;
 *     b / b_lo = parts of B TRANSPOSED, [n,k] with pitch ldb.
 * `epilogue_hash` names a program registered with dalib200_compile that is
 * 'space 2 0' over [m, n] and reads the accumulator through `acc`; its arrays,
 * offsets, strides ((row, col) element strides per array, NULL = contiguous
 * [m,n]) and scalars are passed as for dalib200_launch.  bf16 epilogue arrays
 * are declared 'arg i bf16 E'.  device < 0 only compiles.
 * Replaces cublasSgemm plus the separate kernel the reference runs on the
 * product (dali/array/gemm/cublas_gemm.cu:157-178, dali/array/op/dot.h:7).
 * Returns DALIB200_ERR_UNSUPPORTED for layouts TMA cannot address (use
 * dalib200_gemm and dalib200_launch then). */
int dalib200_gemm_fused(int device, void* stream, int ab_dtype,
                        int64_t m, int64_t n, int64_t k,
                        const void* a, int64_t lda, const void* b, int64_t ldb,
                        const void* a_lo, const void* b_lo,
                        uint64_t epilogue_hash,
                        void* const* array_data, const int64_t* offsets,
                        const int64_t* const* strides, int n_arrays,
                        const void* const* scalars, int n_scalars);

/* Column slices.  An epilogue program may read `acc q` for q < S (S = 2 or 4, fp32
 * operands): its space is then [m, n] and `acc q` at (row, col) is the product's
 * column q*n + col, so B has S*n columns.  One output element sees S accumulator
 * values -- the four gates of an LSTM unit -- and the product itself is never
 * written: the reference materialises dot(x,Wx) + dot(h,Wh) + b as a [B,4H] array
 * and reads it back through four column slices (layers/lstm.cpp:226-263). */
/* The same with the accumulator summed over n_pairs (1 or 2) operand pairs,
 *     acc[m,n] = A_0[m,k_0] . B_0[k_0,n] + A_1[m,k_1] . B_1[k_1,n],
 * in ONE launch and one accumulator: dot(x,Wx) + dot(h,Wh) of a recurrent cell
 * without concatenating anything in memory (the K blocks of the second pair
 * simply follow those of the first in the kernel's pipeline).  Arrays of
 * n_pairs entries; a_lo / b_lo may be NULL (fp32 operands are then split in
 * pool temporaries) and otherwise follow dalib200_gemm_fused. */
int dalib200_gemm_fused_sum(int device, void* stream, int ab_dtype, int n_pairs,
                            int64_t m, int64_t n, const int64_t* k,
                            const void* const* a, const int64_t* lda,
                            const void* const* b, const int64_t* ldb,
                            const void* const* a_lo, const void* const* b_lo,
                            uint64_t epilogue_hash,
                            void* const* array_data, const int64_t* offsets,
                            const int64_t* const* strides, int n_arrays,
                            const void* const* scalars, int n_scalars);

/* hi = x with the 13 low mantissa bits cleared (what TF32 keeps), lo = x - hi,
 * for a rows x cols fp32 matrix with row pitch ld; hi / lo are written tight:
 * [rows, cols], or with transpose != 0 [cols, rows] (the form the B operand is
 * consumed in).  16-byte aligned pointers, cols and ld multiples of 4 (rows too
 * when transposing). */
int dalib200_gemm_split_tf32(int device, void* stream, const float* x,
                             int64_t rows, int64_t cols, int64_t ld, int transpose, float* hi, float* lo);
/* The same for TWO operands of one shape in a single launch, without transposition
 * (the x and h of a recurrent cell, split anew every step). */
int dalib200_gemm_split_tf32_pair(int device, void* stream, const float* x0, const float* x1,
                                  int64_t rows, int64_t cols, int64_t ld0, int64_t ld1,
                                  float* hi0, float* lo0, float* hi1, float* lo1);

/* Synchronises `device` and reads the word tensor-core kernels raise when one of
 * their bounded waits expires (0 = none; 1 producer, 2 MMA issuer, 3 epilogue);
 * a non-zero word is cleared by the read. */
int dalib200_gemm_error_flag(int device, int* flag);

/* Name of the GEMM kernel the last dalib200_gemm* call on this thread chose
 * ("simt", "tcgen05.bf16", "tcgen05.tf32x3", ...); for tests and profiles. */
size_t dalib200_last_gemm_kernel(char* buffer, size_t capacity);

/* ---- running reductions ----------------------------------------------------
 * Replaces the reference's AxisScan node (op::cumsum / op::cumprod / op::axis_scan,
 * dali/array/op/scan.cpp:19-180, kernels :47-140): a running sum / product / max /
 * min along every row of a row-major [rows, cols] matrix (unit inner stride, row
 * pitches in elements).  inclusive != 0: out is [rows, cols].  inclusive == 0:
 * out is [rows, cols + 1], out[r][0] is the reducer's neutral element (0, 1,
 * lowest, max) and out[r][i + 1] the inclusive value at i (scan.cpp:9-15).
 * dtype f32 / f64 / i32.  in and out must not overlap. */
enum dalib200_scan_op { DALIB200_SCAN_SUM = 0, DALIB200_SCAN_PROD = 1, DALIB200_SCAN_MAX = 2, DALIB200_SCAN_MIN = 3 };
int dalib200_scan(int device, void* stream, int dtype, int op, int inclusive,
                  int64_t rows, int64_t cols, const void* in, int64_t in_row_stride,
                  void* out, int64_t out_row_stride);

/* ---- allocation-free entry point ----------------------------------------------
 * No counterpart in the reference (it allocates freely through memory::bank).
 *
 * *out = sum of the n fp32 elements at x (device pointers), asynchronous on
 * `stream` -- the all-axis reduction of dalib200_launch, for callers that may
 * not allocate device memory at call time: a latency-critical host thread that
 * must stay away from allocator locks and driver calls that can block, an
 * embedding with a memory budget fixed at load time.  The cross-CTA
 * exchange space lives in a fixed 8.25 KiB array inside the library image
 * (every GPU that loads the library holds it until exit); the call performs no
 * cudaMalloc / cudaFree and calls no allocating library routine.
 *   - n may be at most DALIB200_NOALLOC_MAX_ELEMENTS; more is refused with
 *     DALIB200_ERR_TOO_LARGE (use dalib200_launch, whose scratch grows).
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress) with that device current; make that first call
 *     before starting any stream capture.
 *   - All calls share the one array: two calls whose kernels can overlap on the
 *     GPU (different streams, no dependency) race on it.  Issue them on one
 *     stream or order them with events.
 * Needs dalib200_init to have bound `device`. */
#define DALIB200_NOALLOC_MAX_ELEMENTS ((int64_t)1 << 31)
int dalib200_sum_f32_noalloc(int device, void* stream, const float* x, int64_t n, float* out);

/* ---- ranks and collectives ------------------------------------------------------
 * One process per GPU, every process holding one shard of the batch (row) dimension.
 * The reference has a slot per GPU in every buffer
 * (dali/array/memory/synchronized_memory.h:46-49) but places each node on one device
 * by a heuristic (dali/array/jit/jit.cpp:367-385) and cannot move data between GPUs
 * (dali/array/memory/memory_ops.cu.cpp:120-125 asserts); these entry points are what
 * replaces that heuristic: shards meet only where a reduction crosses the sharded
 * dimension, in an all-reduce of the partial results.
 *
 * Set-up: rank 0 obtains an id with dalib200_comm_unique_id and hands its bytes to the
 * other ranks by whatever means the launcher offers (torch.distributed, MPI, a file);
 * every rank then calls dalib200_comm_init_rank (collective, blocking).  Payloads of up
 * to 256 KiB per rank then travel as plain stores into peer memory over NVLink with a
 * bounded wait (transport "nccl+peer"; a wait that expires after DALI_B200_PEER_WAIT_MS,
 * default 10000, raises the word read by dalib200_comm_error_flag), larger ones and
 * everything else through NCCL.  dalib200_comm_init_host instead runs every collective
 * through caller-supplied functions on HOST buffers (device buffers are staged through
 * page-locked memory): any fabric, and what the CPU tests use.  world == 1 needs no id. */
#define DALIB200_COMM_ID_BYTES 128
enum dalib200_reduce_op { DALIB200_OP_SUM = 0, DALIB200_OP_PROD = 1, DALIB200_OP_MAX = 2, DALIB200_OP_MIN = 3 };
typedef int (*dalib200_host_allreduce_fn)(void* ctx, void* buf, int64_t n, int dtype, int op);       /* in place; 0 = ok */
typedef int (*dalib200_host_allgather_fn)(void* ctx, const void* send, void* recv, int64_t bytes);   /* recv: world * bytes */
int dalib200_comm_unique_id(void* id /* DALIB200_COMM_ID_BYTES */);
int dalib200_comm_init_rank(int device, int world, int rank, const void* id);
int dalib200_comm_init_host(int world, int rank, dalib200_host_allreduce_fn allreduce,
                            dalib200_host_allgather_fn allgather, void* ctx);
int dalib200_comm_destroy(void);
int dalib200_comm_world(void);                       /* 0 without a communicator */
int dalib200_comm_rank(void);                        /* -1 without a communicator */
/* "none", "single", "nccl+peer", "nccl (<why the peer mapping is off>)", "host" */
size_t dalib200_comm_transport(char* buffer, size_t capacity);
/* Synchronises the communicator's device and reads the word a peer-exchange kernel raises
 * when a rank did not arrive in time (0 = none); a non-zero word is cleared by the read. */
int dalib200_comm_error_flag(int* flag);
/* [lo, hi) of rank's contiguous share of n rows; the first n % world ranks hold one more. */
int dalib200_shard_range(int64_t n, int rank, int world, int64_t* lo, int64_t* hi);
/* buf[i] = op over the ranks of buf[i], in place, the same bits on every rank (contributions
 * are folded in rank order).  dtype f32 / f64 / i32.  Asynchronous on `stream`; device < 0
 * with the host transport: `buf` is host memory.  Every rank must call the collectives in
 * the same order. */
int dalib200_allreduce(int device, void* stream, void* buf, int64_t n, int dtype, int op);
/* The combine of a sharded argmax / argmin: per element the extreme of `values` over the
 * ranks (op max or min) and, in `indices`, the index that came with it; among equal values
 * the lowest index wins, as in the reference's strict-improvement loop
 * (dali/array/jit/all_reduce_kernel_utils.cpp:123-140).  Indices are global (each rank has
 * added its shard's offset).  In place. */
int dalib200_arg_allreduce(int device, void* stream, void* values, int32_t* indices, int64_t n, int dtype, int op);
/* For tests on a box with fewer GPUs than ranks: runs the peer-exchange protocol of the two
 * calls above `repeats` times with `world` (<= 8) virtual ranks inside ONE cooperative kernel
 * on one device.  bufs / indices: host arrays of `world` device pointers (indices may be NULL
 * when arg == 0).  *error_flag receives whether a wait expired. */
int dalib200_peer_emulate(int device, void* stream, int world, int dtype, int op, int arg, void* const* bufs,
                          int32_t* const* indices, int64_t n, int repeats, int* error_flag);

/* ---- page-locked host memory -------------------------------------------------
 * Host buffers the GPUs reach by DMA (cudaHostAlloc, portable across the bound devices): inputs handed over
 * with dali_array_borrow_host and results read with dali_array_to_host move without a staging copy.  The
 * reference stages every transfer through pageable memory (memory_ops.cu.cpp:77-118). */
int dalib200_host_alloc(size_t bytes, void** out);
int dalib200_host_free(void* ptr);

/* ---- device memory ---------------------------------------------------------
 * Replaces memory::bank::allocate / deposit / clear
 * (dali/array/memory/memory_bank.cpp:41-81) and memory::copy / clear
 * (dali/array/memory/memory_ops.cu.cpp:77-131), with 64-bit byte counts.     */
int dalib200_alloc(int device, size_t bytes, void** out);
int dalib200_free(int device, void* ptr, size_t bytes);      /* returns the block to the pool */
int dalib200_pool_clear(int device);                        /* cudaFree everything pooled */
int dalib200_memcpy_h2d(int device, void* dst, const void* src, size_t bytes, void* stream);
int dalib200_memcpy_d2h(int device, void* dst, const void* src, size_t bytes, void* stream);
int dalib200_memcpy_d2d(int device, void* dst, const void* src, size_t bytes, void* stream);
int dalib200_memset(int device, void* dst, int byte, size_t bytes, void* stream);
int dalib200_sync(int device, void* stream);                /* stream == (void*)-1: whole device */

#ifdef __cplusplus
}
#endif
#endif /* DALI_B200_H */
