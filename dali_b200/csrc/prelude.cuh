// Device-side prelude spliced in front of every generated kernel (compiled by
// NVRTC for sm_100a; no host headers are available there).
//
// Functors restate dali/array/functor.h:27-495 as the reference's CPU path
// evaluates them (EXP_F = std::exp etc., functor.h:16-23); int32 operands go
// through double and truncate back, as the templates there do when
// instantiated with R = int.  Reducers restate dali/array/jit/reducer_kernels.h:
// 58-170 (initial values -FLT_MAX / FLT_MAX / 0 / 1, :10-54).

typedef long long i64;
typedef unsigned int u32;
#define DEV __device__ __forceinline__
#define DALI_F32_MAX 3.402823466e+38f
#define DALI_F64_MAX 1.7976931348623158e+308
#define DALI_I32_MAX 2147483647
#define DALI_I32_MIN (-2147483647 - 1)
#define DALI_EPS 1e-6

// bf16 as a STORAGE type of kernel arguments (the reference has float, double and int32 only, dali/array/dtype.h:6-10):
// a load yields the exact float, a store rounds to nearest even (NaN stays NaN); all arithmetic is fp32.
struct bf16_t {
    unsigned short bits;
    DEV bf16_t() {}
    DEV explicit bf16_t(float f) {
        unsigned u = __float_as_uint(f);
        if ((u & 0x7fffffffu) > 0x7f800000u) { bits = (unsigned short)((u >> 16) | 0x0040u); return; }
        u += 0x7fffu + ((u >> 16) & 1u);
        bits = (unsigned short)(u >> 16);
    }
    DEV explicit bf16_t(double f) : bf16_t((float)f) {}
    DEV explicit bf16_t(int f) : bf16_t((float)f) {}
    DEV operator float() const { return __uint_as_float((unsigned)bits << 16); }
};
// the value a bf16 store would keep, as a float (x.astype(bf16) inside a larger expression)
DEV float f_bf16_round(float a) { return (float)bf16_t(a); }
// The two parts of an fp32 value that the 3xTF32 product multiplies: hi keeps the 10 mantissa bits TF32 carries (the low
// 13 cleared), lo = a - hi is exact in fp32 and zero for an infinite a (inf - inf would be NaN).  Same arithmetic as the
// stand-alone split kernels of the GEMM path.
DEV float f_tf32_hi(float a) { return __uint_as_float(__float_as_uint(a) & 0xffffe000u); }
DEV float f_tf32_lo(float a) { const float h = f_tf32_hi(a); return fabsf(h) == __int_as_float(0x7f800000) ? 0.0f : a - h; }
DEV double f_tf32_hi(double a) { return (double)f_tf32_hi((float)a); }
DEV double f_tf32_lo(double a) { return (double)f_tf32_lo((float)a); }
DEV int f_tf32_hi(int a) { return a; }
DEV int f_tf32_lo(int a) { return 0; }

// ---------------------------------------------------------------- functors
template <typename T> DEV T f_identity(T a) { return a; }
template <typename T> DEV T f_negate(T a) { return -a; }
template <typename T> DEV T f_square(T a) { return a * a; }
template <typename T> DEV T f_cube(T a) { return a * a * a; }
template <typename T> DEV T f_add(T a, T b) { return a + b; }
template <typename T> DEV T f_subtract(T a, T b) { return a - b; }
template <typename T> DEV T f_eltmul(T a, T b) { return a * b; }
template <typename T> DEV T f_eltdiv(T a, T b) { return a / b; }
template <typename T> DEV T f_equals(T a, T b) { return a == b ? (T)1 : (T)0; }
template <typename T> DEV T f_fill(T a, T b) { return b; }
// the select of the reference's Diag kernel, "i == j ? diag[j] : 0" (dali/array/op/eye.cpp:33-38), as a functor
template <typename T> DEV T f_where_nonzero(T a, T b) { return a != (T)0 ? b : (T)0; }
template <typename T> DEV T f_div_grad(T a, T b) { return a / (b * b); }
template <typename T> DEV T f_threshold(T a, T b) { return a < b ? (T)1 : (T)0; }
template <typename T> DEV T f_max_scalar(T a, T b) { return a > b ? a : b; }
template <typename T> DEV T f_min_scalar(T a, T b) { return a < b ? a : b; }
template <typename T> DEV T f_lessthanequal(T a, T b) { return a <= b ? (T)1 : (T)0; }
template <typename T> DEV T f_greaterthanequal(T a, T b) { return a >= b ? (T)1 : (T)0; }
template <typename T> DEV T f_dsigmoid(T a) { return a * ((T)1 - a); }
template <typename T> DEV T f_relu(T a) { return a > (T)0 ? a : (T)0; }
template <typename T> DEV T f_relu_backward(T a) { return a > (T)0 ? (T)1 : (T)0; }
template <typename T> DEV T f_sign(T a) { return a > (T)0 ? (T)1 : (T)-1; }
template <typename T> DEV T f_clipped_relu(T x, T c) { return x > (T)0 ? (x > c ? c : x) : (T)0; }
template <typename T> DEV T f_clipped_relu_backward(T x, T c) { return x > (T)0 ? (x > c ? (T)0 : (T)1) : (T)0; }
template <typename T> DEV T f_clip(T x, T c) { return x > c ? c : (x < -c ? -c : x); }
template <typename T> DEV T f_prelu(T x, T w) { return x > (T)0 ? x : w * x; }
template <typename T> DEV T f_prelu_backward_weights(T x, T g) { return x > (T)0 ? (T)0 : x * g; }
template <typename T> DEV T f_prelu_backward_inputs(T x, T w) { return x > (T)0 ? (T)1 : w; }
template <typename T> DEV T f_steep_sigmoid_backward(T x, T a) { return a * (x - x * x); }

DEV float f_abs(float a) { return fabsf(a); }
DEV double f_abs(double a) { return fabs(a); }
DEV int f_abs(int a) { return a < 0 ? -a : a; }

DEV float f_sqrt_f(float a) { return sqrtf(a); }
DEV double f_sqrt_f(double a) { return sqrt(a); }
DEV int f_sqrt_f(int a) { return (int)sqrt((double)a); }

DEV float f_rsqrt(float a) { return (float)(1.0 / (double)sqrtf(a)); }
DEV double f_rsqrt(double a) { return 1.0 / sqrt(a); }
DEV int f_rsqrt(int a) { return (int)(1.0 / sqrt((double)a)); }

DEV float f_inv(float a) { return 1.0f / a; }
DEV double f_inv(double a) { return 1.0 / a; }
DEV int f_inv(int a) { return 1 / a; }

// exp and sigmoid in fp32 go straight to the special-function unit:
// exp(a) = ex2.approx(a * log2(e)).  The rounding of the product contributes a
// relative error of |a| * 6e-8 and ex2.approx 2 ulp, i.e. <= 5.5e-6 over the
// whole finite range (|a| < 88.7) -- inside the 1e-5 fp32 parity bound -- at 2
// instructions instead of the 7-8 of expf().  Denormal results flush to zero.
// The fused chain and softmax kernels are bound by instruction issue and the
// special-function pipe, not by HBM, with the libdevice versions.
DEV float fast_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
DEV float fast_rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
// 1 / y for y in [1, 2^127) on the FMA pipe: an exponent-flipping first guess (at most 5.06 % off), one cubic step
// r += r (e + e^2), e = 1 - y r (error e^3 = 1.3e-4) and one Newton step r += r e (error squared): within 7.7e-8
// relative over every mantissa.  A fused chain whose every element needs two ex2 and a reciprocal is bound by the
// special-function unit (16 lanes per SM per clock); taking the reciprocal off that unit leaves two operations per
// element on it.  (DALI_RCP_MUFU: the special-function reciprocal instead, one instruction; DALI_RCP_TWO_CUBIC: a second
// cubic step in place of the Newton step, one more instruction for 6.0e-8.)
DEV float rcp_ge1(float y) {
#ifdef DALI_RCP_MUFU
    return fast_rcp(y);
#else
    float r = __int_as_float(0x7EF311C7 - __float_as_int(y));
    float e = fmaf(-y, r, 1.0f);
    r = fmaf(r, fmaf(e, e, e), r);
    e = fmaf(-y, r, 1.0f);
#ifdef DALI_RCP_TWO_CUBIC
    return fmaf(r, fmaf(e, e, e), r);
#else
    return fmaf(r, e, r);
#endif
#endif
}
DEV float f_exp(float a) { return fast_ex2(a * 1.4426950408889634f); }
DEV double f_exp(double a) { return exp(a); }
DEV int f_exp(int a) { return (int)exp((double)a); }

DEV float f_log(float a) { return logf(a); }
DEV double f_log(double a) { return log(a); }
DEV int f_log(int a) { return (int)log((double)a); }

DEV float f_negative_log(float a) { return -logf(a); }
DEV double f_negative_log(double a) { return -log(a); }
DEV int f_negative_log(int a) { return (int)(-log((double)a)); }

DEV float f_log_or_zero(float a) { return a > 0.0f ? logf(a) : 0.0f; }
DEV double f_log_or_zero(double a) { return a > 0.0 ? log(a) : 0.0; }
DEV int f_log_or_zero(int a) { return a > 0 ? (int)log((double)a) : 0; }

DEV float f_safe_entropy_log(float a) {
    const float lo = (float)DALI_EPS, hi = (float)(1.0 - DALI_EPS);
    a = a > hi ? hi : a;
    a = a < lo ? lo : a;
    return logf(a);
}
DEV double f_safe_entropy_log(double a) {
    const double lo = DALI_EPS, hi = 1.0 - DALI_EPS;
    a = a > hi ? hi : a;
    a = a < lo ? lo : a;
    return log(a);
}
DEV int f_safe_entropy_log(int a) { return (int)f_safe_entropy_log((double)a); }

// 1 / (1 + exp(-a)): the denominator is in [1, inf], where the approximate
// reciprocal is within 1 ulp and needs no slow path.
// (the exponent is clamped so that 1 + 2^t stays finite; the clamp is min.NaN, one instruction that keeps a NaN operand
// NaN as the reference's 1 / (1 + exp(-a)) does: fminf would return the other operand)
#ifdef DALI_SIGMOID_SELECT
DEV float sigmoid_exponent(float t) { return t > 126.0f ? 126.0f : t; }
#else
DEV float sigmoid_exponent(float t) { float y; asm("min.NaN.f32 %0, %1, 0f42FC0000;" : "=f"(y) : "f"(t)); return y; }
#endif
DEV float f_sigmoid(float a) { return rcp_ge1(1.0f + fast_ex2(sigmoid_exponent(a * -1.4426950408889634f))); }
DEV double f_sigmoid(double a) { return 1.0 / (1.0 + exp(-a)); }
DEV int f_sigmoid(int a) { return (int)(1.0 / (1.0 + exp((double)-a))); }

DEV float f_steep_sigmoid(float x, float g) { return rcp_ge1(1.0f + fast_ex2(sigmoid_exponent((-g * x) * 1.4426950408889634f))); }
DEV double f_steep_sigmoid(double x, double g) { return 1.0 / (1.0 + exp(-g * x)); }
DEV int f_steep_sigmoid(int x, int g) { return (int)(1.0 / (1.0 + exp((double)(-g * x)))); }

DEV float f_tanh(float a) { return tanhf(a); }
DEV double f_tanh(double a) { return tanh(a); }
DEV int f_tanh(int a) { return (int)tanh((double)a); }

DEV float f_dtanh(float a) { return 1.0f - a * a; }
DEV double f_dtanh(double a) { return 1.0 - a * a; }
DEV int f_dtanh(int a) { return 1 - a * a; }

DEV float f_inverse_tanh(float a) { return (logf(1.0f + a) - logf(1.0f - a)) * 0.5f; }
DEV double f_inverse_tanh(double a) { return (log(1.0 + a) - log(1.0 - a)) * 0.5; }
DEV int f_inverse_tanh(int a) { return (int)((log(1.0 + a) - log(1.0 - a)) * 0.5); }

DEV float f_power(float a, float b) { return powf(a, b); }
DEV double f_power(double a, double b) { return pow(a, b); }
DEV int f_power(int a, int b) { return (int)pow((double)a, (double)b); }

DEV float f_softplus(float x) { return x > 20.0f ? x : logf(1.0f + expf(x)); }
DEV double f_softplus(double x) { return x > 20.0 ? x : log(1.0 + exp(x)); }
DEV int f_softplus(int x) { return x > 20 ? x : (int)log(1.0 + exp((double)x)); }

DEV float f_softplus_backward(float x) { if (x > 20.0f) return 1.0f; float e = expf(x); return e / (1.0f + e); }
DEV double f_softplus_backward(double x) { if (x > 20.0) return 1.0; double e = exp(x); return e / (1.0 + e); }
DEV int f_softplus_backward(int x) { return (int)f_softplus_backward((double)x); }

DEV float f_isnotanumber(float a) { return isnan(a) ? 1.0f : 0.0f; }
DEV double f_isnotanumber(double a) { return isnan(a) ? 1.0 : 0.0; }
DEV int f_isnotanumber(int a) { return 0; }
DEV float f_isinfinity(float a) { return isinf(a) ? 1.0f : 0.0f; }
DEV double f_isinfinity(double a) { return isinf(a) ? 1.0 : 0.0; }
DEV int f_isinfinity(int a) { return 0; }

DEV float f_binary_cross_entropy(float x, float t) { return -(t * logf(x) + (1.0f - t) * logf(1.0f - x)); }
DEV double f_binary_cross_entropy(double x, double t) { return -(t * log(x) + (1.0 - t) * log(1.0 - x)); }
DEV int f_binary_cross_entropy(int x, int t) { return (int)f_binary_cross_entropy((double)x, (double)t); }
DEV float f_binary_cross_entropy_grad(float x, float t) { return (t - x) / (x * (x - 1.0f)); }
DEV double f_binary_cross_entropy_grad(double x, double t) { return (t - x) / (x * (x - 1.0)); }
DEV int f_binary_cross_entropy_grad(int x, int t) { return (int)f_binary_cross_entropy_grad((double)x, (double)t); }

// functor::round is floor(a + 0.5), functor::ceil is ceil(a); both convert.
template <typename R> DEV R f_round(float a) { return (R)floorf(a + 0.5f); }
template <typename R> DEV R f_round(double a) { return (R)floor(a + 0.5); }
template <typename R> DEV R f_round(int a) { return (R)a; }
template <typename R> DEV R f_ceiling(float a) { return (R)ceilf(a); }
template <typename R> DEV R f_ceiling(double a) { return (R)ceil(a); }
template <typename R> DEV R f_ceiling(int a) { return (R)a; }

// ---------------------------------------------------------------- reducers
template <typename T> struct Lim;
template <> struct Lim<float> { static DEV float lo() { return -DALI_F32_MAX; } static DEV float hi() { return DALI_F32_MAX; } };
template <> struct Lim<double> { static DEV double lo() { return -DALI_F64_MAX; } static DEV double hi() { return DALI_F64_MAX; } };
template <> struct Lim<int> { static DEV int lo() { return DALI_I32_MIN; } static DEV int hi() { return DALI_I32_MAX; } };

struct RSum { template <typename T> static DEV T init() { return (T)0; } template <typename T> static DEV T apply(T a, T b) { return a + b; } };
struct RProd { template <typename T> static DEV T init() { return (T)1; } template <typename T> static DEV T apply(T a, T b) { return a * b; } };
struct RMax {
    template <typename T> static DEV T init() { return Lim<T>::lo(); }
    template <typename T> static DEV T apply(T a, T b) { return a > b ? a : b; }
    static DEV float apply(float a, float b) { return fmaxf(a, b); }
    template <typename T> static DEV bool better(T a, T b) { return a > b; }
    // the larger of two candidates with a NaN never winning (fmaxf / fmax / integer max): what arg-reductions use to
    // ask of a whole group of elements at once whether any of them beats the running value
    template <typename T> static DEV T pick(T a, T b) { return a > b ? a : b; }
    static DEV float pick(float a, float b) { return fmaxf(a, b); }
    static DEV double pick(double a, double b) { return fmax(a, b); }
};
struct RMin {
    template <typename T> static DEV T init() { return Lim<T>::hi(); }
    template <typename T> static DEV T apply(T a, T b) { return a < b ? a : b; }
    static DEV float apply(float a, float b) { return fminf(a, b); }
    template <typename T> static DEV bool better(T a, T b) { return a < b; }
    template <typename T> static DEV T pick(T a, T b) { return a < b ? a : b; }
    static DEV float pick(float a, float b) { return fminf(a, b); }
    static DEV double pick(double a, double b) { return fmin(a, b); }
};

// (value, index) for argmax / argmin.  The reference keeps the FIRST index at
// which the running value strictly improves (tmp != res after Reduce,
// dali/array/jit/all_reduce_kernel_utils.cpp:123-140,210-223) and starts from
// index 0: `take` reproduces that for one element, `merge` for two partial
// results (equal values -> lower index).
template <typename T> struct ArgPair { T v; i64 i; };
template <typename Op, typename T> DEV ArgPair<T> arg_init() { ArgPair<T> p; p.v = Op::template init<T>(); p.i = 0; return p; }
template <typename Op, typename T> DEV void arg_take(ArgPair<T>& acc, T v, i64 i) {
    if (Op::better(v, acc.v)) { acc.v = v; acc.i = i; }
}
template <typename Op, typename T> DEV ArgPair<T> arg_merge(ArgPair<T> a, ArgPair<T> b) {
    const bool take_b = Op::better(b.v, a.v) || (b.v == a.v && b.i < a.i);
    return take_b ? b : a;
}

// Loads that bypass L1: partial results written by other CTAs of the same launch.
template <typename T> DEV T ld_cg(const T* p) { return __ldcg(p); }
template <typename T> DEV ArgPair<T> ld_cg(const ArgPair<T>* p) {
    ArgPair<T> r;
    r.v = __ldcg(&p->v);
    r.i = __ldcg(&p->i);
    return r;
}

template <typename T> DEV T shfl_xor(T v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
template <typename T> DEV ArgPair<T> shfl_xor(ArgPair<T> p, int m) {
    ArgPair<T> q;
    q.v = __shfl_xor_sync(0xffffffffu, p.v, m);
    q.i = __shfl_xor_sync(0xffffffffu, p.i, m);
    return q;
}

// Butterfly over the W (<= 32, power of two) adjacent lanes of a warp that
// share a row; every lane ends with the result.
template <typename Op, int W, typename T> DEV T group_reduce(T v) {
#pragma unroll
    for (int m = W / 2; m > 0; m >>= 1) v = Op::apply(v, shfl_xor(v, m));
    return v;
}
template <typename Op, int W, typename T> DEV ArgPair<T> group_arg_reduce(ArgPair<T> v) {
#pragma unroll
    for (int m = W / 2; m > 0; m >>= 1) v = arg_merge<Op, T>(v, shfl_xor(v, m));
    return v;
}

// Reduction over the T threads that share a row.  T <= 32: shuffles only.
// T > 32: one partial per warp through shared memory (`buf` holds NT/32
// entries and must not be reused before the next __syncthreads), then every
// thread folds its row's T/32 partials in warp order -- deterministic.
template <typename Op, int T_, typename T> DEV T row_reduce(T v, T* buf) {
    if (T_ <= 32) return group_reduce<Op, (T_ <= 32 ? T_ : 32)>(v);
    v = group_reduce<Op, 32>(v);
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) buf[warp] = v;
    __syncthreads();
    const int first = (warp / (T_ / 32)) * (T_ / 32);
    T r = buf[first];
#pragma unroll
    for (int k = 1; k < T_ / 32; ++k) r = Op::apply(r, buf[first + k]);
    return r;
}
template <typename Op, int T_, typename T> DEV ArgPair<T> row_arg_reduce(ArgPair<T> v, ArgPair<T>* buf) {
    if (T_ <= 32) return group_arg_reduce<Op, (T_ <= 32 ? T_ : 32)>(v);
    v = group_arg_reduce<Op, 32>(v);
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) buf[warp] = v;
    __syncthreads();
    const int first = (warp / (T_ / 32)) * (T_ / 32);
    ArgPair<T> r = buf[first];
#pragma unroll
    for (int k = 1; k < T_ / 32; ++k) r = arg_merge<Op, T>(r, buf[first + k]);
    return r;
}

// A row shared by the CTAs of a thread-block cluster (the row skeleton's `cluster` variant): every CTA reduces its
// slice of the columns, stores the partial result into slot [its rank] of EVERY CTA of the cluster through distributed
// shared memory, the cluster meets at its hardware barrier (no spinning: the CTAs of a cluster are co-scheduled), and
// every CTA folds the slots in rank order -- the same order everywhere, so all CTAs continue with the same bits.
DEV unsigned cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
DEV void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <typename T> DEV void cluster_store(T* local_slot, unsigned target, const T& v) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(local_slot)), "r"(target));
    const unsigned* w = reinterpret_cast<const unsigned*>(&v);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(T) / 4); ++i)
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote + 4u * i), "r"(w[i]) : "memory");
}
template <typename Op, int CL, typename T> DEV T cluster_fold(T partial, T* slots, unsigned rank) {
    if (threadIdx.x < CL) cluster_store(&slots[rank], threadIdx.x, partial);
    cluster_barrier();
    T r = slots[0];
#pragma unroll
    for (int q = 1; q < CL; ++q) r = Op::apply(r, slots[q]);
    return r;
}
template <typename Op, int CL, typename T> DEV ArgPair<T> cluster_arg_fold(ArgPair<T> partial, ArgPair<T>* slots, unsigned rank) {
    if (threadIdx.x < CL) cluster_store(&slots[rank], threadIdx.x, partial);
    cluster_barrier();
    ArgPair<T> r = slots[0];
#pragma unroll
    for (int q = 1; q < CL; ++q) r = arg_merge<Op, T>(r, slots[q]);
    return r;
}

// Whole-CTA reduction (NT threads, NT a multiple of 32); result valid in every
// thread.  `buf` holds NT/32 entries.
template <typename Op, int NT, typename T> DEV T block_reduce(T v, T* buf) { return row_reduce<Op, NT>(v, buf); }
template <typename Op, int NT, typename T> DEV ArgPair<T> block_arg_reduce(ArgPair<T> v, ArgPair<T>* buf) { return row_arg_reduce<Op, NT>(v, buf); }

// Atomics for scatter-assign through gather (the reference maps = += -= to
// atomicExch / atomicAdd, dali/array/op/gather.cpp:14-28).
DEV void atomic_add(float* p, float v) { atomicAdd(p, v); }
DEV void atomic_add(double* p, double v) { atomicAdd(p, v); }
DEV void atomic_add(int* p, int v) { atomicAdd(p, v); }
DEV void atomic_exch(float* p, float v) { atomicExch(p, v); }
DEV void atomic_exch(int* p, int v) { atomicExch(p, v); }
DEV void atomic_exch(double* p, double v) { atomicExch((unsigned long long*)p, (unsigned long long)__double_as_longlong(v)); }

// First statement of every generated kernel.  Kernels are launched as programmatic dependents: their CTAs may
// become resident while the kernel before them in the stream is still draining; nothing may touch global memory
// before that kernel has completed (griddepcontrol.wait), and the kernel after this one is allowed to line up
// the same way from here on.  Without the launch attribute both instructions do nothing.
DEV void kernel_entry() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Rows staged through shared memory by bulk asynchronous copies (the row skeleton's `stage` variant): one mbarrier
// per ring slot counts the bytes of the copies that fill it.
DEV unsigned stage_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
DEV void stage_bar_init(unsigned long long* bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(stage_smem(bar))); }
// makes the initialised barriers visible to the copy engine
DEV void stage_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// orders this thread's (and, after __syncwarp, its warp's) reads of a slot before the copy engine's next write to it
DEV void stage_fence_reuse() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
DEV void stage_expect(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(stage_smem(bar)), "r"(bytes) : "memory");
}
// global -> shared, 16-byte aligned on both sides, a multiple of 16 bytes; local memory only, no multicast
DEV void stage_copy(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(stage_smem(dst)), "l"(src), "r"(bytes), "r"(stage_smem(bar)) : "memory");
}
// Waits for the slot's copies.  Bounded (about a second): a copy from valid memory always completes, so giving up only
// keeps a kernel with a defect from spinning for ever; the row is then processed with whatever the slot holds.
DEV void stage_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok = 0;
    const long long t0 = clock64();
    while (true) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(stage_smem(bar)), "r"(parity) : "memory");
        if (ok || clock64() - t0 > 2000000000LL) return;
    }
}

// 128-bit global access; callers guarantee 16-byte alignment.
template <typename T, int N> struct alignas(sizeof(T) * N) Vec { T x[N]; };
template <typename T, int N> DEV Vec<T, N> vload(const T* p) { return *reinterpret_cast<const Vec<T, N>*>(p); }
template <typename T, int N> DEV void vstore(T* p, const Vec<T, N>& v) { *reinterpret_cast<Vec<T, N>*>(p) = v; }
// the same as a streaming store (evict-first in L2): for outputs that are not read again while something else should stay cached
template <typename T, int N> DEV void vstore_stream(T* p, const Vec<T, N>& v) {
    if (sizeof(T) * N == 16) __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&v));
    else if (sizeof(T) * N == 8) __stcs(reinterpret_cast<uint2*>(p), *reinterpret_cast<const uint2*>(&v));
    else *reinterpret_cast<Vec<T, N>*>(p) = v;
}

// Counter-based random numbers: Philox4x32-10 (Salmon et al., SC'11) with counter = (block, 0, 0, 0)
// and key = (seed, 0); which block and words an element reads is stated at RngBlock below.  Replaces the thrust generators the reference seeds per
// call on the GPU (dali/array/op/random.cu.cpp:153-232): being a pure function of (index,
// seed) it fuses into whatever consumes the numbers (a dropout mask never touches memory) and
// gives the same stream whatever the launch geometry.
DEV void philox4x32_10(unsigned c0, unsigned k0, unsigned out[4]) {
    unsigned c1 = 0, c2 = 0, c3 = 0, k1 = 0;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const unsigned n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
// Element i of a random array reads the Philox block and the words that its type needs:
//   fp32 uniform            block i >> 2, word i & 3
//   fp64 uniform, fp32 normal   block i >> 1, words 2 (i & 1) and 2 (i & 1) + 1
//   fp64 normal             block i, all four words
// so neighbouring elements share a block.  RngBlock keeps the last block of one random node across the lanes of a
// thread's vector: four fp32 uniforms cost one Philox call (when the vector starts on a block boundary; two otherwise).
struct RngBlock { unsigned id; unsigned w[4]; int valid; };
DEV void rng_fetch(RngBlock& b, unsigned id, int seed) {
    if (!b.valid || b.id != id) {
        philox4x32_10(id, (unsigned)seed, b.w);
        b.id = id;
        b.valid = 1;
    }
}
DEV unsigned rng_word(const RngBlock& b, int k) { return k == 0 ? b.w[0] : (k == 1 ? b.w[1] : (k == 2 ? b.w[2] : b.w[3])); }
DEV double rng_u53(unsigned hi, unsigned lo) { return (double)(hi >> 5) * 67108864.0 + (double)(lo >> 6); }
// u in [0, 1): 24 bits for float, 53 for double
template <typename T> DEV T f_rng_uniform(int index, int seed, RngBlock& b);
template <> DEV float f_rng_uniform<float>(int index, int seed, RngBlock& b) {
    rng_fetch(b, (unsigned)index >> 2, seed);
    return (float)(rng_word(b, index & 3) >> 8) * (1.0f / 16777216.0f);
}
template <> DEV double f_rng_uniform<double>(int index, int seed, RngBlock& b) {
    rng_fetch(b, (unsigned)index >> 1, seed);
    const int k = (index & 1) * 2;
    return rng_u53(rng_word(b, k), rng_word(b, k + 1)) * (1.0 / 9007199254740992.0);
}
// standard normal by Box-Muller on two uniforms of one Philox block: sqrt(-2 ln u1) cos(2 pi u2), u1 in (0, 1]
template <typename T> DEV T f_rng_normal(int index, int seed, RngBlock& b);
template <> DEV float f_rng_normal<float>(int index, int seed, RngBlock& b) {
    rng_fetch(b, (unsigned)index >> 1, seed);
    const int k = (index & 1) * 2;
    const float u1 = ((float)(rng_word(b, k) >> 8) + 1.0f) * (1.0f / 16777216.0f);
    const float u2 = (float)(rng_word(b, k + 1) >> 8) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}
template <> DEV double f_rng_normal<double>(int index, int seed, RngBlock& b) {
    rng_fetch(b, (unsigned)index, seed);
    const double u1 = (rng_u53(b.w[0], b.w[1]) + 1.0) * (1.0 / 9007199254740992.0);
    const double u2 = rng_u53(b.w[2], b.w[3]) * (1.0 / 9007199254740992.0);
    return sqrt(-2.0 * log(u1)) * cospi(2.0 * u2);
}
// one element on its own (row-level statements, GEMM epilogues)
template <typename T> DEV T f_rng_uniform(int index, int seed) { RngBlock b = {0u, {0u, 0u, 0u, 0u}, 0}; return f_rng_uniform<T>(index, seed, b); }
template <typename T> DEV T f_rng_normal(int index, int seed) { RngBlock b = {0u, {0u, 0u, 0u, 0u}, 0}; return f_rng_normal<T>(index, seed, b); }

// An argument with no memory behind it whose "element" at offset i is base + i: with the
// per-dim strides every argument has, base + sum(index_d * stride_d) is any affine function
// of the iteration index (what the reference's arange / one_hot / diag kernels read from
// `query`, dali/array/op/arange.cpp:41, one_hot.cpp:45, eye.cpp:37).
struct IotaPtr {
    i64 base;
    DEV int operator[](i64 i) const { return (int)(base + i); }
    DEV IotaPtr operator+(i64 i) const { return IotaPtr{base + i}; }
};
template <typename T, int N> DEV Vec<T, N> vload(IotaPtr p) {
    Vec<T, N> v;
#pragma unroll
    for (int j = 0; j < N; ++j) v.x[j] = (T)(p.base + j);
    return v;
}
