/* dali_b200 -- C binding of the lazy Array / op:: front end.
 *
 * One function per member of the reference's public C++ API on the hot path
 * (class Array, dali/array/array.h:18-260; namespace op, dali/array/op.h:1-26),
 * over opaque handles, so that the same lazy-expression -> optimize -> compile
 * -> cache -> run flow can be driven from any language with a C FFI (the tests
 * and bench.py use it through ctypes).  C++ callers use the headers under
 * dali_b200/host/include directly.
 *
 * Every function returns 0 or a negative dalib200_status; the message is read
 * with dalib200_last_error() (include/dali_b200.h).  Handles are created by
 * the functions that return one through an out parameter and are released
 * with dali_array_free().  Nothing computes until dali_array_eval(),
 * dali_array_to_host() or dali_array_item() asks for a value.
 */
#ifndef DALI_B200_ARRAY_H
#define DALI_B200_ARRAY_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dali_array_s* dali_array_t;

/* ---- construction (Array::Array, Array::adopt_buffer, array.h:43-73) ------------- */
/* copies `data` (C-contiguous, `shape`) into a new host-fresh Array; dtype as dalib200_dtype */
int dali_array_from_host(const void* data, const int64_t* shape, int ndim, int dtype, dali_array_t* out);
/* wraps HOST memory the caller keeps owning (no copy, never freed here; what the reference's
 * Array::adopt_buffer is used for when a harness hands in prepared inputs, array.cpp:203-222).
 * The memory must stay alive and unchanged until every expression that reads it has been
 * evaluated; page-locked memory reaches the GPU by DMA without a staging copy. */
int dali_array_borrow_host(void* data, const int64_t* shape, int ndim, int dtype, dali_array_t* out);
/* Not in the reference: evaluates several lazy arrays of one shape in ONE kernel when their trees are elementwise
 * (shared sub-expressions are computed once, every array is stored), one after the other otherwise. */
int dali_array_eval_together(const dali_array_t* arrays, int n, int wait);
/* NumPy .npy files, the reference's on-disk format (Array::load / Array::save, array.cpp:253-359): float32,
 * float64 and int32, C or Fortran order on load (a Fortran-ordered file comes back as a transposed view),
 * C order on save. */
int dali_array_load(const char* path, dali_array_t* out);
int dali_array_save(const char* path, dali_array_t a);
/* wraps DEVICE memory the caller keeps owning (no copy, never freed here) */
int dali_array_from_device(void* device_ptr, const int64_t* shape, int ndim, int dtype, int gpu, dali_array_t* out);
int dali_array_empty(const int64_t* shape, int ndim, int dtype, dali_array_t* out);
int dali_array_zeros(const int64_t* shape, int ndim, int dtype, dali_array_t* out);
int dali_array_scalar(double value, int dtype, dali_array_t* out);
int dali_array_arange(int start, int stop, int step, dali_array_t* out);
int dali_array_free(dali_array_t a);

/* ---- inspection (array.h:104-124) ------------------------------------------------- */
int dali_array_ndim(dali_array_t a);
int dali_array_dtype(dali_array_t a);
int dali_array_shape(dali_array_t a, int64_t* shape_out);          /* ndim entries */
int dali_array_is_buffer(dali_array_t a);                           /* 1 once evaluated */
size_t dali_array_expression_name(dali_array_t a, char* buffer, size_t capacity);   /* full_expression_name() */

/* ---- evaluation (Array::eval, array.cpp:232-245; scalar casts :88-105) ------------- */
int dali_array_eval(dali_array_t a, int wait);
/* evaluates, then copies the elements in C order into `out` (capacity in bytes) */
int dali_array_to_host(dali_array_t a, void* out, size_t capacity);
/* evaluates a one-element Array and returns it as double (operator double()) */
int dali_array_item(dali_array_t a, double* out);
/* device pointer of an evaluated, contiguous Array (readonly access on `gpu`) */
int dali_array_device_ptr(dali_array_t a, int gpu, void** out);

/* ---- views (array.h:126-170) ------------------------------------------------------- */
int dali_array_index(dali_array_t a, int axis, int idx, dali_array_t* out);                     /* pluck_axis(axis, idx) */
int dali_array_slice(dali_array_t a, int axis, int start, int stop, int step, dali_array_t* out);   /* pluck_axis(axis, Slice) */
int dali_array_expand_dims(dali_array_t a, int axis, dali_array_t* out);
int dali_array_squeeze(dali_array_t a, int axis, dali_array_t* out);
int dali_array_transpose(dali_array_t a, const int* axes, int n_axes, dali_array_t* out);      /* n_axes = 0: reverse */
int dali_array_broadcast_to(dali_array_t a, const int64_t* shape, int ndim, dali_array_t* out);
int dali_array_reshape(dali_array_t a, const int64_t* shape, int ndim, dali_array_t* out);
int dali_array_astype(dali_array_t a, int dtype, dali_array_t* out);

/* ---- op:: (dali/array/op/unary.h, binary.h, reducers.h, gather.h, softmax.h, dot.h) -- */
int dali_op_unary(const char* name, dali_array_t a, dali_array_t* out);      /* "exp", "sigmoid", ... */
int dali_op_binary(const char* name, dali_array_t a, dali_array_t b, dali_array_t* out);   /* "add", "eltmul", ... */
/* name: sum prod max min mean L2_norm; n_axes < 0 reduces over all axes */
int dali_op_reduce(const char* name, dali_array_t a, const int* axes, int n_axes, int keepdims, dali_array_t* out);
/* name: argmax argmin; all_axes != 0 ignores `axis` */
int dali_op_argreduce(const char* name, dali_array_t a, int axis, int all_axes, dali_array_t* out);
int dali_op_gather(dali_array_t source, dali_array_t indices, dali_array_t* out);
int dali_op_gather_from_rows(dali_array_t source, dali_array_t indices, dali_array_t* out);
/* op/eye.h, op/one_hot.h, op/outer.h, op/scan.h, op/arange.h: all lazy; reducer = sum | prod | max | min */
int dali_op_diag(dali_array_t diag, int rows, int cols, dali_array_t* out);
int dali_op_one_hot(dali_array_t indices, int depth, dali_array_t on_value, dali_array_t off_value, dali_array_t* out);
int dali_op_outer(dali_array_t a, dali_array_t b, dali_array_t* out);
/* op/concatenate.h:7-9: the arrays one after another along `axis` (hstack = axis -1, vstack = axis 0) */
int dali_op_concatenate(const dali_array_t* arrays, int n, int axis, dali_array_t* out);
int dali_op_scan(dali_array_t a, const char* reducer, int inclusive, dali_array_t* out);
int dali_op_arange(dali_array_t start, dali_array_t stop, dali_array_t step, dali_array_t* out);
/* op/random.h: kind = uniform (a = low, b = high) | normal (a = loc, b = scale) | bernoulli | bernoulli_normalized
 * (a = prob, b ignored); utils::random::set_seed (dali/utils/random.h:39) */
int dali_op_random(const char* kind, dali_array_t a, dali_array_t b, const int64_t* shape, int ndim, dali_array_t* out);
int dali_random_set_seed(int seed);
int dali_op_softmax(dali_array_t logits, int axis, dali_array_t* out);
int dali_op_dot(dali_array_t a, dali_array_t b, dali_array_t* out);

/* ---- assignment (array.h:201-205, 233-241): op 0 '=', 1 '+=', 2 '-=', 3 '*=', 4 '/=', 5 '<<=' */
int dali_array_assign(dali_array_t dest, int op, dali_array_t value);

/* memory::default_preferred_device = Device::gpu(gpu) (dali/runtime_config.cpp:12-18): where
 * newly created Arrays compute.  One process per GPU sets its own index. */
int dali_set_default_device(int gpu);

/* ---- sharding over the ranks of the communicator (include/dali_b200.h, "ranks and collectives").  Not in the
 * reference, whose device placement is a per-node heuristic (dali/array/jit/jit.cpp:367-385).
 * set_shard declares an evaluated array to be rows [lo, lo + extent) of a logical array of `total` rows along
 * `axis` (axis < 0 removes the mark); the mark travels with everything derived from the array, and a reduction over
 * that axis or a product that contracts it combines the ranks' partial results.  scatter_rows keeps this rank's rows
 * (dalib200_shard_range) of a C-contiguous host array and marks them. */
int dali_array_set_shard(dali_array_t a, int axis, int64_t lo, int64_t total);
int dali_array_get_shard(dali_array_t a, int* axis, int64_t* lo, int64_t* total);
int dali_array_scatter_rows(const void* data, const int64_t* global_shape, int ndim, int dtype, dali_array_t* out);
/* number of cross-rank combines this thread's evaluations have issued and a description of the last one */
size_t dali_lazy_collectives(int64_t* count, char* buffer, size_t capacity);

/* ---- trace scopes (dali/utils/scope.h:11-57): every computation opens a scope named after the expression it
 * evaluates (dali/array/expression/computation.cpp:14-21); the compile-or-load step a scope "get_function"
 * (dali/array/jit/jit.cpp:1015).  start begins recording, stop ends it and returns the names of the scopes that were
 * left in between, one per line -- what dali/array/tests/dot_tests.cpp:17-35 counts to show that evaluating a product
 * runs exactly one computation. */
int dali_scope_trace_start(void);
size_t dali_scope_trace_stop(char* buffer, size_t capacity);

/* ---- introspection of the lowering, for tests (kernels, gemms, temporaries launched by
 * this thread so far) and the IR / kernel variant of the last fused kernel ----------- */
int dali_lazy_stats(int64_t counts[3]);
/* on != 0: evaluations on this thread lower, register and NVRTC-compile their kernels but
 * allocate, copy and launch nothing (results undefined).  Shows what fuses without a GPU. */
int dali_lazy_set_dry_run(int on);
size_t dali_lazy_last_ir(char* buffer, size_t capacity);
size_t dali_lazy_last_variant(char* buffer, size_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* DALI_B200_ARRAY_H */
