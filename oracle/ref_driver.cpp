// Test infrastructure only -- not part of the shipped library.
//
// Command-line driver around the REFERENCE's own CPU implementation of the
// hot path (built by oracle/build_ref.sh into oracle/_ref/libdali_ref.so).
// It is written against the reference's public API (class Array,
// dali/array/array.h:18-230; op::*, dali/array/op.h:1-26) and is used
//   * to pin the C restatement in oracle/dali_oracle.c,
//   * to generate the golden fixtures under tests/golden/, and
//   * as the timed CPU baseline ("kind": "reference") of bench.py.
//
// usage: ref_driver <cache-dir> <case> <args...>   (arrays are .npy files)
//   unary   <name> in out            binary <name> a b out
//   reduce  <sum|prod|max|min|mean|l2|argmax|argmin> <axis|all> in out [reps]
//   softmax in out [reps]            (op::softmax composition, axis -1)
//   softmax_naive in out [reps]      (the expression spelled out by the caller)
//   lstm    x h c Wx Wh b c_out h_out [reps]
//   gemm_tanh A B bias out [reps]    (fp32: the reference has no bf16)
//   dot     a b out [reps]
//   chain   x w b out [reps]         sum(sigmoid(x*w+b)*exp(-x*x))
//   gather  src idx out              gather_rows src idx out
//   scatter_add dest idx out         (dest[idx] += 1, result = dest)
//   arange  <i32|f32|f64> start stop step out     (numbers on the command line)
//   diag_scalar <i32|f32|f64> value rows cols out  diag_vec d rows cols out
//   one_hot idx depth on off out     (on / off: doubles on the command line, as the reference's test passes them)
//   outer   a b out                  scan <sum|prod> <0|1 inclusive> in out [reps]
// Every timed case prints "TIME_MS first=<ms> best=<ms> reps=<n>".
#include "dali/array/array.h"
#include "dali/array/op.h"
#include "dali/array/op/softmax.h"
#include "dali/array/op/arange.h"
#include "dali/array/op/eye.h"
#include "dali/array/op/one_hot.h"
#include "dali/array/op/outer.h"
#include "dali/array/op/scan.h"
#include "dali/utils/random.h"
#include "dali/utils/compiler.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <iostream>
#include <map>
#include <string>

#ifdef REF_DRIVER_BOUND
extern "C" void dali_b200_binding_stats(int* launched, int* fell_back);
extern "C" int dali_b200_binding_gemms();
#endif

typedef std::chrono::steady_clock clk;
static double ms(clk::time_point a, clk::time_point b) {
    return std::chrono::duration<double, std::milli>(b - a).count();
}

// run f once (JIT compile / cache load included), then `reps` more times;
// prints the first, the best and every repeat so callers can drop warm-ups
static void timed(int reps, const std::function<void()>& f) {
    auto t0 = clk::now(); f(); auto t1 = clk::now();
    double best = ms(t0, t1);
    bool any = false;
    std::string all;
    for (int r = 0; r < reps; ++r) {
        auto a = clk::now(); f(); auto b = clk::now();
        double t = ms(a, b);
        if (!any || t < best) best = t;
        any = true;
        char buf[64];
        std::snprintf(buf, sizeof buf, " %.6f", t);
        all += buf;
    }
    std::printf("TIME_MS first=%.6f best=%.6f reps=%d\n", ms(t0, t1), best, reps);
    std::printf("TIMES_MS%s\n", all.c_str());
}

static Array load(const char* path) {
    Array a = Array::load(std::string(path));
    a.eval();
    return a;
}

static void save(const char* path, const Array& a) {
    // the reference's npy writer does not take rank-0 arrays: store scalars as shape {1}
    // (and it crashes on an evaluated node that is not a plain buffer, which is
    // what op::gather leaves behind: copy those through an identity first)
    Array out = a;
    out.eval();
    if (!out.is_buffer()) { out = op::identity(out); out.eval(); }
    if (out.ndim() == 0) out = out.reshape({1});
    Array::save(std::string(path), out);
}

typedef Array (*unary_fn)(Array);
typedef Array (*binary_fn)(Array, Array);

static std::map<std::string, unary_fn> unary_table() {
    std::map<std::string, unary_fn> t;
    t["identity"] = op::identity; t["sqrt"] = op::sqrt; t["square"] = op::square;
    t["abs"] = op::abs; t["sigmoid"] = op::sigmoid; t["dsigmoid"] = op::dsigmoid;
    t["tanh"] = op::tanh; t["dtanh"] = op::dtanh; t["relu"] = op::relu;
    t["relu_backward"] = op::relu_backward; t["eltinv"] = op::eltinv; t["exp"] = op::exp;
    t["log"] = op::log; t["log_or_zero"] = op::log_or_zero; t["sign"] = op::sign;
    t["softplus"] = op::softplus; t["softplus_backward"] = op::softplus_backward;
    t["cube"] = op::cube; t["rsqrt"] = op::rsqrt; t["isnan"] = op::isnan; t["isinf"] = op::isinf;
    t["inverse_tanh"] = op::inverse_tanh;
    return t;
}

static std::map<std::string, binary_fn> binary_table() {
    std::map<std::string, binary_fn> t;
    t["add"] = op::add; t["subtract"] = op::subtract; t["eltmul"] = op::eltmul;
    t["eltdiv"] = op::eltdiv; t["equals"] = op::equals; t["pow"] = op::pow;
    t["steep_sigmoid"] = op::steep_sigmoid; t["steep_sigmoid_backward"] = op::steep_sigmoid_backward;
    t["clipped_relu"] = op::clipped_relu; t["clipped_relu_backward"] = op::clipped_relu_backward;
    t["prelu"] = op::prelu; t["prelu_backward_weights"] = op::prelu_backward_weights;
    t["prelu_backward_inputs"] = op::prelu_backward_inputs;
    t["lessthanequal"] = op::lessthanequal; t["greaterthanequal"] = op::greaterthanequal;
    t["maximum"] = op::maximum; t["minimum"] = op::minimum; t["clip"] = op::clip;
    t["binary_cross_entropy"] = op::binary_cross_entropy;
    t["binary_cross_entropy_grad"] = op::binary_cross_entropy_grad;
    return t;
}

static int usage() {
    std::fprintf(stderr, "usage: ref_driver <cache-dir> <case> <args...>\n");
    return 2;
}

int main(int argc, char** argv) {
    if (argc < 3) return usage();
    memory::WithDevicePreference dp(memory::Device::cpu());
    std::string cache(argv[1]);
    if (cache.empty() || cache[cache.size() - 1] != '/') cache += "/";
    array_op_compiler.set_output_path(cache);
    std::string c(argv[2]);
    char** a = argv + 3;
    int n = argc - 3;
    auto reps_at = [&](int i) { return n > i ? std::atoi(a[i]) : 0; };

    if (c == "unary" && n >= 3) {
        auto t = unary_table();
        if (!t.count(a[0])) { std::fprintf(stderr, "unknown unary %s\n", a[0]); return 2; }
        Array x = load(a[1]);
        Array y = t[a[0]](x); y.eval();
        save(a[2], y);
    } else if (c == "binary" && n >= 4) {
        auto t = binary_table();
        if (!t.count(a[0])) { std::fprintf(stderr, "unknown binary %s\n", a[0]); return 2; }
        Array l = load(a[1]), r = load(a[2]);
        Array y = t[a[0]](l, r); y.eval();
        save(a[3], y);
    } else if (c == "reduce" && n >= 4) {
        std::string opn(a[0]), ax(a[1]);
        Array x = load(a[2]);
        Array out;
        bool all = ax == "all";
        int axis = all ? 0 : std::atoi(a[1]);
        timed(reps_at(4), [&]() {
            Array r;
            if (opn == "sum") r = all ? op::sum(x) : op::sum(x, {axis});
            else if (opn == "prod") r = all ? op::prod(x) : op::prod(x, {axis});
            else if (opn == "max") r = all ? op::max(x) : op::max(x, {axis});
            else if (opn == "min") r = all ? op::min(x) : op::min(x, {axis});
            else if (opn == "mean") r = all ? op::mean(x) : op::mean(x, {axis});
            else if (opn == "l2") r = all ? op::L2_norm(x) : op::L2_norm(x, {axis});
            else if (opn == "argmax") r = all ? op::argmax(x) : op::argmax(x, axis);
            else if (opn == "argmin") r = all ? op::argmin(x) : op::argmin(x, axis);
            else { std::fprintf(stderr, "unknown reducer %s\n", opn.c_str()); std::exit(2); }
            r.eval();
            out = r;
        });
        save(a[3], out);
    } else if ((c == "softmax" || c == "softmax_naive") && n >= 2) {
        Array x = load(a[0]);
        Array out;
        timed(reps_at(2), [&]() {
            Array r;
            if (c == "softmax") {
                r = op::softmax(x, -1);
            } else {
                Array exped = op::exp(x - op::max(x, {-1}, true));
                r = exped / op::sum(exped, {-1}, true);
            }
            r.eval();
            out = r;
        });
        save(a[1], out);
    } else if (c == "lstm" && n >= 8) {
        Array x = load(a[0]), h = load(a[1]), cc = load(a[2]);
        Array Wx = load(a[3]), Wh = load(a[4]), b = load(a[5]);
        int H = cc.shape()[1];
        Array c_new, h_new;
        timed(reps_at(8), [&]() {
            Array gates = op::dot(x, Wx) + op::dot(h, Wh) + b;
            Array i = op::sigmoid(gates[Slice()][Slice(0, H)]);
            Array f = op::sigmoid(gates[Slice()][Slice(H, 2 * H)]);
            Array o = op::sigmoid(gates[Slice()][Slice(2 * H, 3 * H)]);
            Array g = op::tanh(gates[Slice()][Slice(3 * H, 4 * H)]);
            Array cn = f * cc + i * g;
            Array hn = o * op::tanh(cn);
            hn.eval();
            cn.eval();
            c_new = cn; h_new = hn;
        });
        save(a[6], c_new);
        save(a[7], h_new);
    } else if (c == "gemm_tanh" && n >= 4) {
        Array A = load(a[0]), B = load(a[1]), bias = load(a[2]);
        Array out;
        timed(reps_at(4), [&]() {
            Array r = op::tanh(op::dot(A, B) + bias[Broadcast()]);
            r.eval();
            out = r;
        });
        save(a[3], out);
    } else if (c == "dot" && n >= 3) {
        Array A = load(a[0]), B = load(a[1]);
        Array out;
        timed(reps_at(3), [&]() { Array r = op::dot(A, B); r.eval(); out = r; });
        save(a[2], out);
    } else if (c == "chain" && n >= 4) {
        Array x = load(a[0]);
        float w = (float)std::atof(a[1]), b = (float)std::atof(a[2]);
        Array out;
        timed(reps_at(4), [&]() {
            Array y = op::sigmoid(x * w + b) * op::exp(-x * x);
            Array s = op::sum(y);
            s.eval();
            out = s;
        });
        save(a[3], out);
    } else if (c == "gather" && n >= 3) {
        Array src = load(a[0]), idx = load(a[1]);
        Array r = op::gather(src, idx); r.eval();
        save(a[2], r);
    } else if (c == "gather_rows" && n >= 3) {
        Array src = load(a[0]), idx = load(a[1]);
        Array r = op::gather_from_rows(src, idx); r.eval();
        save(a[2], r);
    } else if (c == "scatter_add" && n >= 3) {
        Array dest = load(a[0]), idx = load(a[1]);
        Array gathered = dest[idx];
        (gathered += 1).eval();
        save(a[2], dest);
    } else if (c == "arange" && n >= 5) {
        std::string t(a[0]);
        auto num = [&](const char* v) {
            return t == "i32" ? Array(std::atoi(v)) : t == "f32" ? Array((float)std::atof(v)) : Array(std::atof(v));
        };
        Array r = op::arange(num(a[1]), num(a[2]), num(a[3])); r.eval();
        save(a[4], r);
    } else if (c == "diag_scalar" && n >= 5) {
        std::string t(a[0]);
        Array d = t == "i32" ? Array(std::atoi(a[1])) : t == "f32" ? Array((float)std::atof(a[1])) : Array(std::atof(a[1]));
        Array r = op::diag(d, std::atoi(a[2]), std::atoi(a[3])); r.eval();
        save(a[4], r);
    } else if (c == "diag_vec" && n >= 4) {
        Array r = op::diag(load(a[0]), std::atoi(a[1]), std::atoi(a[2])); r.eval();
        save(a[3], r);
    } else if (c == "one_hot" && n >= 5) {
        Array r = op::one_hot(load(a[0]), std::atoi(a[1]), std::atof(a[2]), std::atof(a[3])); r.eval();
        save(a[4], r);
    } else if (c == "outer" && n >= 3) {
        Array r = op::outer(load(a[0]), load(a[1])); r.eval();
        save(a[2], r);
    } else if (c == "unary_t" && n >= 3) {
        // y = contiguous copy of f(x)^T: an elementwise tree under a transposing view
        auto t = unary_table();
        if (!t.count(a[0])) { std::fprintf(stderr, "unknown unary %s\n", a[0]); return 2; }
        Array x = load(a[1]);
        Array r;
        timed(reps_at(3), [&]() {
            Array y = t[a[0]](x).transpose().ascontiguousarray();
            y.eval();
            r = y;
        });
        save(a[2], r);
    } else if (c == "scan" && n >= 4) {
        Array x = load(a[2]);
        const bool inclusive = std::atoi(a[1]) != 0, sum = std::string(a[0]) == "sum";
        Array r;
        timed(reps_at(4), [&]() {
            Array s = sum ? op::cumsum(x, inclusive) : op::cumprod(x, inclusive);
            s.eval();
            r = s;
        });
        save(a[3], r);
    } else {
        return usage();
    }
#ifdef REF_DRIVER_BOUND
    // ref_driver_bound (linked against libdali_ref_bound.so): how much of the case the binding took
    int launched = 0, fell_back = 0;
    dali_b200_binding_stats(&launched, &fell_back);
    std::printf("BINDING launched=%d fell_back=%d gemms=%d\n", launched, fell_back, dali_b200_binding_gemms());
#endif
    return 0;
}
