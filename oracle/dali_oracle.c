/* TEST INFRASTRUCTURE ONLY -- never linked into, imported by or shipped with
 * the library.  Only tests/, __graft_entry__.smoke() and the cpu_baseline /
 * --impl reference legs of bench.py may call it, and only as the checker.
 *
 * Plain-C restatement of the reference's CPU algorithm for the hot path
 * (lazy expression -> JIT -> run on memory::Device::cpu()).  Parity is PINNED:
 * tests/golden/make_golden.py ran the reference's own CPU path (oracle/_ref,
 * built from the reference sources by oracle/build_ref.sh) on seeded inputs and
 * committed the outputs as tests/golden/reference_cpu.npz; tests/test_oracle.py
 * checks every function here against those fixtures (bit for bit where the
 * arithmetic is the reference's own) and against the known-answer cases of the
 * reference's own suite
 * (dali/array/tests/tests.cpp:1120-1361, dali/array/tests/dot_tests.cpp:10-118).
 *
 * What each function follows:
 *   functors      dali/array/functor.h:27-495 with the CPU macro set
 *                 (EXP_F = std::exp ..., functor.h:16-23)
 *   reductions    the sequential loops emitted by
 *                 dali/array/jit/all_reduce_kernel_utils.cpp:105-121 (all),
 *                 :142-154 (axis) with reducers::{sum,product,maximum,minimum}
 *                 (dali/array/jit/reducer_kernels.h:58-170, init values :10-54)
 *   arg-reduce    all_reduce_kernel_utils.cpp:123-140, 210-223 (first strict
 *                 improvement wins)
 *   softmax       dali/array/op/softmax.cpp:5-8 evaluated as the reference
 *                 does: temporaries for the row max, exp(a - max) and its row sum
 *   gather        dali/array/op/gather.cpp:45-65, gather_from_rows.cpp:53-78
 *   scan          dali/array/op/scan.cpp:47-77 (left-to-right running reduction)
 *   one_hot, diag dali/array/op/one_hot.cpp:41-46, eye.cpp:33-38
 *   gemm          row-major C = A.B as dali/array/gemm/cpu_gemm.cpp:22-84 asks
 *                 of CBLAS; here with a double accumulator (CBLAS itself is a
 *                 third-party dependency with no pinned version, so only the
 *                 reference's small exact known answers pin it)
 */
#include <float.h>
#include <limits.h>
#include <math.h>
#include <tgmath.h>   /* exp/log/tanh pick float or double by operand type, like the C++ overloads */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ functors */
/* Each functor is written once over a macro parameter R and instantiated for
 * float, double and int, mirroring template<typename R> struct X { Map }.    */

#define EPS 1e-6

#define DEFINE_FUNCTORS(R, SUF, EXP, LOG, TANH, POW)                                              \
    static R square_##SUF(R a) { return a * a; }                                                  \
    static R cube_##SUF(R a) { return a * a * a; }                                                \
    static R identity_##SUF(R a) { return a; }                                                    \
    static R negate_##SUF(R a) { return -a; }                                                     \
    static R inv_##SUF(R a) { return ((R)1.0) / a; }                                              \
    static R sigmoid_##SUF(R a) { return (R)(1.0 / (1.0 + EXP(-a))); }                            \
    static R dsigmoid_##SUF(R a) { return a * (((R)1.0) - a); }                                   \
    static R log_##SUF(R a) { return (R)LOG(a); }                                                 \
    static R negative_log_##SUF(R a) { return (R)(-LOG(a)); }                                     \
    static R safe_entropy_log_##SUF(R a) {                                                        \
        R s = a; const R lo = (R)EPS; const R hi = (R)(1.0 - EPS);                                \
        if (s > hi) s = hi; if (s < lo) s = lo; return (R)LOG(s); }                               \
    static R exp_##SUF(R a) { return (R)EXP(a); }                                                 \
    static R dtanh_##SUF(R a) { return (R)(1.0 - a * a); }                                        \
    static R inverse_tanh_##SUF(R a) { return (R)((LOG(1 + a) - LOG(1 - a)) * 0.5); }             \
    static R log_or_zero_##SUF(R a) { return a > 0 ? (R)LOG(a) : (R)0; }                          \
    static R sign_##SUF(R a) { return (R)(a > 0.0 ? 1.0 : -1.0); }                                \
    static R relu_##SUF(R a) { return (R)(a > 0.0 ? a : 0.0); }                                   \
    static R relu_backward_##SUF(R a) { return (R)(a > 0.0 ? 1.0 : 0.0); }                        \
    static R softplus_##SUF(R a) { return a > 20.0 ? a : (R)LOG((R)1.0 + EXP(a)); }               \
    static R softplus_backward_##SUF(R a) {                                                       \
        return a > 20.0 ? (R)1.0 : (R)(EXP(a) / ((R)1.0 + EXP(a))); }                             \
    static R add_##SUF(R a, R b) { return a + b; }                                                \
    static R subtract_##SUF(R a, R b) { return a - b; }                                           \
    static R eltmul_##SUF(R a, R b) { return a * b; }                                             \
    static R eltdiv_##SUF(R a, R b) { return a / b; }                                             \
    static R equals_##SUF(R a, R b) { return a == b ? 1 : 0; }                                    \
    static R fill_##SUF(R a, R b) { (void)a; return b; }                                          \
    static R div_grad_##SUF(R a, R b) { return a / (b * b); }                                     \
    static R threshold_##SUF(R a, R b) { return (R)(a < b ? 1.0 : 0.0); }                         \
    static R max_scalar_##SUF(R a, R b) { return a > b ? a : b; }                                 \
    static R min_scalar_##SUF(R a, R b) { return a < b ? a : b; }                                 \
    static R power_##SUF(R a, R b) { return (R)POW(a, b); }                                       \
    static R steep_sigmoid_##SUF(R x, R g) { return (R)(1.0 / (1.0 + EXP(-g * x))); }             \
    static R steep_sigmoid_backward_##SUF(R x, R g) { return g * (x - x * x); }                   \
    static R clipped_relu_##SUF(R x, R c) { return (R)(x > 0.0 ? (x > c ? c : x) : 0.0); }        \
    static R clipped_relu_backward_##SUF(R x, R c) {                                              \
        return (R)(x > 0.0 ? (x > c ? 0.0 : 1.0) : 0.0); }                                        \
    static R clip_##SUF(R x, R c) { return x > c ? c : (x < -c ? -c : x); }                       \
    static R lessthanequal_##SUF(R x, R u) { return x <= u ? 1 : 0; }                             \
    static R greaterthanequal_##SUF(R x, R l) { return x >= l ? 1 : 0; }                          \
    static R binary_cross_entropy_##SUF(R x, R t) {                                               \
        R d1 = (R)(t * LOG(x)); R d0 = (R)((1.0 - t) * LOG(1. - x)); return -(d1 + d0); }         \
    static R binary_cross_entropy_grad_##SUF(R x, R t) {                                          \
        R num = t - x; R den = (R)(x * (x - 1.0)); return num / den; }                            \
    static R prelu_##SUF(R x, R w) { return x > 0 ? x : w * x; }                                  \
    static R prelu_backward_weights_##SUF(R x, R g) { return x > 0 ? 0 : x * g; }                 \
    static R prelu_backward_inputs_##SUF(R x, R w) { return (R)(x > 0 ? 1.0 : w); }

/* CPU macro set: std::exp / std::log / std::tanh pick the float overload for
 * float operands and the double one for double and int operands -- also
 * inside one functor (binary_cross_entropy takes log of a float and of a
 * double); <tgmath.h> reproduces that overload choice in C. */
DEFINE_FUNCTORS(float, f32, exp, log, tanh, powf)
DEFINE_FUNCTORS(double, f64, exp, log, tanh, pow)
DEFINE_FUNCTORS(int, i32, exp, log, tanh, pow)

/* specialisations (functor.h:93-123, 266-276, 320-325, 208-239) */
static float sqrt_f_f32(float a) { return (float)sqrt((double)a); }
static double sqrt_f_f64(double a) { return sqrt(a); }
static int sqrt_f_i32(int a) { return (int)sqrt((double)a); }
/* unqualified sqrt() in namespace functor resolves to ::sqrt(double) */
static float rsqrt_f32(float a) { return (float)(1.0 / sqrt((double)a)); }
static double rsqrt_f64(double a) { return 1.0 / sqrt(a); }
static int rsqrt_i32(int a) { return (int)(1.0 / sqrt((double)a)); }
static float tanh_f32(float a) { return tanhf(a); }
static double tanh_f64(double a) { return tanh(a); }
static int tanh_i32(int a) { return (int)tanh((double)a); }
static float abs_f32(float a) { return fabsf(a); }
static double abs_f64(double a) { return fabs(a); }
static int abs_i32(int a) { return abs(a); }
static float isnotanumber_f32(float a) { return (float)(isnan(a) ? 1 : 0); }
static double isnotanumber_f64(double a) { return (double)(isnan(a) ? 1 : 0); }
static int isnotanumber_i32(int a) { (void)a; return 0; }
static float isinfinity_f32(float a) { return (float)(isinf(a) ? 1 : 0); }
static double isinfinity_f64(double a) { return (double)(isinf(a) ? 1 : 0); }
static int isinfinity_i32(int a) { (void)a; return 0; }

#define UNARY_LIST(X)                                                                              \
    X(square) X(cube) X(identity) X(negate) X(inv) X(sigmoid) X(dsigmoid) X(log) X(negative_log)   \
    X(safe_entropy_log) X(exp) X(dtanh) X(inverse_tanh) X(log_or_zero) X(sign) X(relu)             \
    X(relu_backward) X(softplus) X(softplus_backward) X(sqrt_f) X(rsqrt) X(tanh) X(abs)            \
    X(isnotanumber) X(isinfinity)
#define BINARY_LIST(X)                                                                             \
    X(add) X(subtract) X(eltmul) X(eltdiv) X(equals) X(fill) X(div_grad) X(threshold)              \
    X(max_scalar) X(min_scalar) X(power) X(steep_sigmoid) X(steep_sigmoid_backward)                \
    X(clipped_relu) X(clipped_relu_backward) X(clip) X(lessthanequal) X(greaterthanequal)          \
    X(binary_cross_entropy) X(binary_cross_entropy_grad) X(prelu) X(prelu_backward_weights)        \
    X(prelu_backward_inputs)

/* dtype codes: 0 float, 1 double, 2 int32 (dali/array/dtype.h:6-10) */
int oracle_unary(const char* name, int dtype, const void* x, void* y, int64_t n) {
#define X(N)                                                                                       \
    if (strcmp(name, #N) == 0) {                                                                   \
        if (dtype == 0) { for (int64_t i = 0; i < n; ++i) ((float*)y)[i] = N##_f32(((const float*)x)[i]); }          \
        else if (dtype == 1) { for (int64_t i = 0; i < n; ++i) ((double*)y)[i] = N##_f64(((const double*)x)[i]); }   \
        else { for (int64_t i = 0; i < n; ++i) ((int*)y)[i] = N##_i32(((const int*)x)[i]); }       \
        return 0;                                                                                  \
    }
    UNARY_LIST(X)
#undef X
    return -1;
}

/* b_stride 0 broadcasts a single right operand (scalar operand tests) */
int oracle_binary(const char* name, int dtype, const void* a, const void* b, int64_t b_stride, void* y, int64_t n) {
#define X(N)                                                                                       \
    if (strcmp(name, #N) == 0) {                                                                   \
        if (dtype == 0) { for (int64_t i = 0; i < n; ++i) ((float*)y)[i] = N##_f32(((const float*)a)[i], ((const float*)b)[i * b_stride]); }        \
        else if (dtype == 1) { for (int64_t i = 0; i < n; ++i) ((double*)y)[i] = N##_f64(((const double*)a)[i], ((const double*)b)[i * b_stride]); } \
        else { for (int64_t i = 0; i < n; ++i) ((int*)y)[i] = N##_i32(((const int*)a)[i], ((const int*)b)[i * b_stride]); }                         \
        return 0;                                                                                  \
    }
    BINARY_LIST(X)
#undef X
    return -1;
}

/* functor::round = floor(a + 0.5), functor::cast = R(a) (functor.h:133-147) */
void oracle_round_f32_i32(const float* x, int* y, int64_t n) { for (int64_t i = 0; i < n; ++i) y[i] = (int)floor(x[i] + 0.5); }
void oracle_round_f64_i32(const double* x, int* y, int64_t n) { for (int64_t i = 0; i < n; ++i) y[i] = (int)floor(x[i] + 0.5); }

/* ------------------------------------------------------------------ reductions */
/* View of the operand: rows x cols with element strides; every output row is
 * the left-to-right fold of its cols in the operand's own type, which is what
 * the reference's generated CPU loop does (volatile accumulator, no
 * reassociation).  `kind`: 0 sum 1 product 2 maximum 3 minimum.            */
#define DEFINE_REDUCE(R, SUF, LO, HI)                                                              \
    void oracle_reduce_##SUF(int kind, const R* x, int64_t rows, int64_t cols, int64_t rs,         \
                             int64_t cs, R* out) {                                                 \
        for (int64_t r = 0; r < rows; ++r) {                                                       \
            volatile R res = kind == 0 ? (R)0 : kind == 1 ? (R)1 : kind == 2 ? LO : HI;            \
            const R* p = x + r * rs;                                                               \
            for (int64_t c = 0; c < cols; ++c) {                                                   \
                R v = p[c * cs];                                                                   \
                if (kind == 0) res += v;                                                           \
                else if (kind == 1) res *= v;                                                      \
                else if (kind == 2) res = res > v ? res : v;                                       \
                else res = res < v ? res : v;                                                      \
            }                                                                                      \
            out[r] = res;                                                                          \
        }                                                                                          \
    }                                                                                              \
    /* first index at which the running value strictly improves; starts at 0 */                   \
    void oracle_argreduce_##SUF(int kind, const R* x, int64_t rows, int64_t cols, int64_t rs,      \
                                int64_t cs, int* out) {                                            \
        for (int64_t r = 0; r < rows; ++r) {                                                       \
            R res = kind == 2 ? LO : HI;                                                           \
            int idx = 0;                                                                           \
            const R* p = x + r * rs;                                                               \
            for (int64_t c = 0; c < cols; ++c) {                                                   \
                R tmp = res;                                                                       \
                R v = p[c * cs];                                                                   \
                if (kind == 2) res = res > v ? res : v; else res = res < v ? res : v;              \
                if (tmp != res) idx = (int)c;                                                      \
            }                                                                                      \
            out[r] = idx;                                                                          \
        }                                                                                          \
    }
DEFINE_REDUCE(float, f32, -FLT_MAX, FLT_MAX)
DEFINE_REDUCE(double, f64, -DBL_MAX, DBL_MAX)
DEFINE_REDUCE(int, i32, INT_MIN, INT_MAX)

/* The same fold with a double accumulator, plus sum |x|: the yardstick for
 * floating sums (any summation order is within 1e-5 * sum|x| of it for the
 * sizes used; the reference's own fp32 fold is reported beside it).         */
void oracle_sum_f64acc_f32(const float* x, int64_t rows, int64_t cols, int64_t rs, int64_t cs,
                           double* out, double* out_abs) {
    for (int64_t r = 0; r < rows; ++r) {
        double s = 0, sa = 0;
        const float* p = x + r * rs;
        for (int64_t c = 0; c < cols; ++c) { s += p[c * cs]; sa += fabs(p[c * cs]); }
        out[r] = s;
        if (out_abs) out_abs[r] = sa;
    }
}

/* ------------------------------------------------------------------ softmax */
/* op::softmax over the last axis of a contiguous [rows, cols] float array,
 * staged as the reference evaluates it: max -> exp(a - max) -> sum -> divide. */
void oracle_softmax_f32(const float* a, int64_t rows, int64_t cols, float* out) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* p = a + r * cols;
        float* o = out + r * cols;
        volatile float mx = -FLT_MAX;
        for (int64_t c = 0; c < cols; ++c) mx = mx > p[c] ? mx : p[c];
        volatile float sum = 0;
        for (int64_t c = 0; c < cols; ++c) { o[c] = expf(p[c] - mx); sum += o[c]; }
        for (int64_t c = 0; c < cols; ++c) o[c] = o[c] / sum;
    }
}

/* ------------------------------------------------------------------ gather */
/* out[i, :] = src[idx[i], :]   (row_len = product of the trailing dims) */
void oracle_gather(const void* src, const int* idx, int64_t n_idx, int64_t row_len, int itemsize, void* out) {
    for (int64_t i = 0; i < n_idx; ++i)
        memcpy((char*)out + i * row_len * itemsize, (const char*)src + (int64_t)idx[i] * row_len * itemsize,
               (size_t)(row_len * itemsize));
}
/* out[i, :] = src[i, idx[i], :] */
void oracle_gather_from_rows(const void* src, const int* idx, int64_t rows, int64_t cols, int64_t inner,
                             int itemsize, void* out) {
    for (int64_t i = 0; i < rows; ++i)
        memcpy((char*)out + i * inner * itemsize,
               (const char*)src + ((i * cols + idx[i]) * inner) * itemsize, (size_t)(inner * itemsize));
}
/* dest[idx[i], :] += upd[i, :]  (serial order, as the reference's CPU loop) */
void oracle_scatter_add_f32(float* dest, const int* idx, const float* upd, int64_t n_idx, int64_t row_len) {
    for (int64_t i = 0; i < n_idx; ++i)
        for (int64_t j = 0; j < row_len; ++j) dest[(int64_t)idx[i] * row_len + j] += upd[i * row_len + j];
}
void oracle_scatter_add_i32(int* dest, const int* idx, const int* upd, int64_t n_idx, int64_t row_len) {
    for (int64_t i = 0; i < n_idx; ++i)
        for (int64_t j = 0; j < row_len; ++j) dest[(int64_t)idx[i] * row_len + j] += upd[i * row_len + j];
}

/* ------------------------------------------------------------------ gemm */
/* C[m,n] = A[m,k] . B[k,n], element strides given, double accumulator. */
void oracle_gemm_f32(const float* a, int64_t a_rs, int64_t a_cs, const float* b, int64_t b_rs, int64_t b_cs,
                     float* c, int64_t m, int64_t n, int64_t k) {
    double* acc = (double*)malloc(sizeof(double) * (size_t)n);
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) acc[j] = 0;
        for (int64_t p = 0; p < k; ++p) {
            const double av = a[i * a_rs + p * a_cs];
            const float* bp = b + p * b_rs;
            for (int64_t j = 0; j < n; ++j) acc[j] += av * bp[j * b_cs];
        }
        for (int64_t j = 0; j < n; ++j) c[i * n + j] = (float)acc[j];
    }
    free(acc);
}
void oracle_gemm_i32(const int* a, const int* b, int* c, int64_t m, int64_t n, int64_t k) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            int s = 0;
            for (int64_t p = 0; p < k; ++p) s += a[i * k + p] * b[p * n + j];
            c[i * n + j] = s;
        }
}

/* ------------------------------------------------------------------ fused configs */
/* LSTM cell gating on materialised gates [B, 4H] (columns i | f | o | g),
 * c' = sigmoid(f) * c + sigmoid(i) * tanh(g), h' = sigmoid(o) * tanh(c'),
 * each factor through the float functors above (dali/layers/lstm.cpp:226-263
 * gives the equations; the column layout is this build's choice).           */
void oracle_lstm_gating_f32(const float* gates, const float* c, int64_t B, int64_t H, float* c_new, float* h_new) {
    for (int64_t r = 0; r < B; ++r)
        for (int64_t j = 0; j < H; ++j) {
            const float* g = gates + r * 4 * H;
            float i_ = sigmoid_f32(g[j]), f_ = sigmoid_f32(g[H + j]), o_ = sigmoid_f32(g[2 * H + j]);
            float g_ = tanh_f32(g[3 * H + j]);
            float cn = f_ * c[r * H + j] + i_ * g_;
            c_new[r * H + j] = cn;
            h_new[r * H + j] = o_ * tanh_f32(cn);
        }
}
/* y_i = sigmoid(x_i * w + b) * exp(-x_i * x_i); returns the reference's
 * sequential fp32 sum, the double-accumulated sum and sum |y|.             */
void oracle_chain_sum_f32(const float* x, int64_t n, float w, float b, float* sum_f32, double* sum_f64, double* sum_abs) {
    volatile float s = 0;
    double d = 0, da = 0;
    for (int64_t i = 0; i < n; ++i) {
        float y = sigmoid_f32(x[i] * w + b) * exp_f32(-x[i] * x[i]);
        s += y;
        d += y;
        da += fabs(y);
    }
    *sum_f32 = s;
    *sum_f64 = d;
    *sum_abs = da;
}
/* tanh(x + bias[col]) epilogue of the GEMM config, float functors. */
void oracle_bias_tanh_f32(const float* x, const float* bias, int64_t rows, int64_t cols, float* out) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) out[r * cols + c] = tanh_f32(x[r * cols + c] + bias[c]);
}

/* ---- running reductions: AxisScan, dali/array/op/scan.cpp:47-77 --------------------
 * The CPU body walks each row left to right: so_far = init; for i: so_far = so_far (op) x[i];
 * out = so_far.  Exclusive results start with the neutral element and are one longer.
 * op: 0 sum, 1 prod, 2 max, 3 min; neutral elements as in jit/reducer_kernels.h:10-54. */
#define SCAN_BODY(T, INIT_MAX, INIT_MIN)                                                          \
    for (int64_t r = 0; r < rows; ++r) {                                                          \
        const T* x = (const T*)in + r * cols;                                                     \
        T* y = (T*)out + r * (cols + (inclusive ? 0 : 1));                                        \
        volatile T so_far = op == 0 ? (T)0 : op == 1 ? (T)1 : op == 2 ? (T)(INIT_MAX) : (T)(INIT_MIN); \
        if (!inclusive) *y++ = so_far;                                                            \
        for (int64_t i = 0; i < cols; ++i) {                                                      \
            const T v = x[i];                                                                     \
            if (op == 0) so_far = so_far + v;                                                     \
            else if (op == 1) so_far = so_far * v;                                                \
            else if (op == 2) so_far = so_far > v ? so_far : v;                                   \
            else so_far = so_far < v ? so_far : v;                                                \
            y[i] = so_far;                                                                        \
        }                                                                                         \
    }
int oracle_scan(int op, int dtype, int inclusive, int64_t rows, int64_t cols, const void* in, void* out) {
    if (op < 0 || op > 3) return 1;
    if (dtype == 0) { SCAN_BODY(float, -FLT_MAX, FLT_MAX) }
    else if (dtype == 1) { SCAN_BODY(double, -DBL_MAX, DBL_MAX) }
    else if (dtype == 2) { SCAN_BODY(int, INT_MIN, INT_MAX) }
    else return 1;
    return 0;
}

/* ---- one_hot: dali/array/op/one_hot.cpp:41-46 -----------------------------------------
 * T is_on = indices[...] == d; return on * is_on + (1.0 - is_on) * off   (T = dtype of on_value) */
int oracle_one_hot(const int* idx, int64_t n, int depth, int dtype, double on, double off, void* out) {
    for (int64_t i = 0; i < n; ++i)
        for (int d = 0; d < depth; ++d) {
            if (dtype == 0) { float is_on = idx[i] == d; ((float*)out)[i * depth + d] = (float)((float)on * is_on + (1.0 - is_on) * (float)off); }
            else if (dtype == 1) { double is_on = idx[i] == d; ((double*)out)[i * depth + d] = on * is_on + (1.0 - is_on) * off; }
            else if (dtype == 2) { int is_on = idx[i] == d; ((int*)out)[i * depth + d] = (int)((int)on * is_on + (1.0 - is_on) * (int)off); }
            else return 1;
        }
    return 0;
}

/* ---- diag / eye: dali/array/op/eye.cpp:33-38: query[1] == query[0] ? diag[query[1]] : 0 ----
 * d_len == 0: scalar diag (d points at one element). */
int oracle_diag(int dtype, const void* d, int64_t d_len, int64_t rows, int64_t cols, void* out) {
    const int item = dtype == 1 ? 8 : 4;
    if (dtype < 0 || dtype > 2) return 1;
    memset(out, 0, (size_t)(rows * cols) * item);
    for (int64_t i = 0; i < rows && i < cols; ++i)
        memcpy((char*)out + (i * cols + i) * item, (const char*)d + (d_len ? i : 0) * item, item);
    return 0;
}
