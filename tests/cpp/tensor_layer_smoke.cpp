// The reference's autodiff layer (class Tensor, graph::backward, namespace tensor_ops) running on
// the B200 back end.  This program is linked with the reference's own dali/tensor objects, which
// were compiled UNCHANGED against this back end's Array headers; every forward value and every
// gradient below is therefore computed by reference code calling the lazy Array / op:: API, and
// checked against central finite differences the way the reference's tests do it
// (dali/test_utils.h:277-373 gradient_same: objective = sum of the output, one element of one
// argument moved by +-eps at a time, in double precision).
//
// Each block restates, in this file's own words, what a test of dali/tensor/tests.cpp or
// dali/tensor/op/*_tests.cpp asserts (file:line given).  Needs a GPU.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "dali/array/array.h"
#include "dali/array/op.h"
#include "dali/tensor/op.h"
#include "dali/tensor/solver.h"
#include "dali/tensor/tape.h"
#include "dali/tensor/tensor.h"
#include "dali/utils/random.h"

using std::vector;

static int checks = 0, failures = 0, thrown = 0;
#define CHECK(cond)                                                                   \
    do {                                                                              \
        ++checks;                                                                     \
        if (!(cond)) { ++failures; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)

typedef std::function<Tensor(vector<Tensor>&)> functor_t;

static Tensor uniform(double lo, double hi, const vector<int>& shape) {
    return Tensor::uniform(Array(lo), Array(hi), shape);   // Array(double) is a double scalar
}

// reads a (possibly strided) array into a host vector, row-major
static vector<double> to_host(const Array& a) {
    Array c = a.astype(DTYPE_DOUBLE).ascontiguousarray();
    c.eval();
    const double* p = (const double*)c.memory()->readonly_data(memory::Device::cpu()) + c.offset();
    return vector<double>(p, p + c.number_of_elements());
}

// analytic gradients from the tape against central differences of sum(f(args))
static bool gradient_same_or_throw(const char* name, functor_t f, vector<Tensor> args, double tolerance, double eps,
                                   bool fail_on_zero_gradient);

// one line per case: "case <name>: ok", ": wrong" or ": throws" (a std::runtime_error from the layer or the back end;
// the message goes to a second line that the comparison between back ends ignores)
static bool gradient_same(const char* name, functor_t f, vector<Tensor> args, double tolerance = 1e-5, double eps = 1e-4,
                          bool fail_on_zero_gradient = true) {
    ++checks;
    try {
        const bool ok = gradient_same_or_throw(name, f, args, tolerance, eps, fail_on_zero_gradient);
        std::printf("case %s: %s\n", name, ok ? "ok" : "wrong");
        if (!ok) ++failures;
        return ok;
    } catch (const std::runtime_error& e) {
        graph::clear();
        std::printf("case %s: throws\n  (%s)\n", name, e.what());
        ++thrown;
        return false;
    }
}

static bool gradient_same_or_throw(const char* name, functor_t f, vector<Tensor> args, double tolerance, double eps,
                                   bool fail_on_zero_gradient) {
    graph::clear();
    for (auto& a : args) a.dw.clear();
    Tensor out = f(args);
    out.grad();
    graph::backward();
    bool ok = true;
    for (size_t k = 0; k < args.size() && ok; ++k) {
        Tensor& arg = args[k];
        vector<double> analytic = to_host(arg.dw);
        vector<double> numeric(analytic.size());
        graph::NoBackprop nb;
        bool nonzero = false;
        for (int i = 0; i < arg.number_of_elements(); ++i) {
            const double prev = (double)Array(arg.w(i));
            arg.w(i).assign(prev + eps).eval();
            const double plus = (double)Array(f(args).w.sum());
            arg.w(i).assign(prev - eps).eval();
            const double minus = (double)Array(f(args).w.sum());
            arg.w(i).assign(prev).eval();
            numeric[i] = (plus - minus) / (2.0 * eps);
            nonzero = nonzero || numeric[i] != 0.0;
        }
        double worst = 0.0;
        for (size_t i = 0; i < numeric.size(); ++i) worst = std::max(worst, std::fabs(numeric[i] - analytic[i]));
        if (!(worst <= tolerance)) {
            std::printf("  %s: gradient of argument %zu differs from finite differences by %.3g (tolerance %.3g)\n", name, k + 1,
                        worst, tolerance);
            ok = false;
        }
        if (fail_on_zero_gradient && !nonzero) {
            std::printf("  %s: gradient of argument %zu should not be all zeros\n", name, k + 1);
            ok = false;
        }
    }
    return ok;
}

// dali/tensor/tests.cpp:338-364 TensorUnaryTests: every unary method of Tensor on uniform [2, 3, 4] inputs
// (Tensor::cube is left out: its backward pass in the reference, dali/tensor/op/unary.cpp:19, squares the OUTPUT
// instead of the input, so it disagrees with finite differences on any back end)
static void unary_gradients() {
    utils::random::set_seed(100);
    struct Case { const char* name; std::function<Tensor(const Tensor&)> fn; double lo, hi, tol; bool nonzero; };
    const vector<Case> cases = {
        {"square", [](const Tensor& t) { return t.square(); }, -5.0, 5.0, 1e-3, true},
        {"sqrt", [](const Tensor& t) { return t.sqrt(); }, 0.5, 5.0, 1e-3, true},
        {"eltinv", [](const Tensor& t) { return t.eltinv(); }, 0.5, 5.0, 1e-3, true},
        {"sigmoid", [](const Tensor& t) { return t.sigmoid(); }, -20.0, 20.0, 1e-3, true},
        {"tanh", [](const Tensor& t) { return t.tanh(); }, -20.0, 20.0, 1e-3, true},
        {"softplus", [](const Tensor& t) { return t.softplus(); }, -20.0, 20.0, 1e-2, true},
        {"log", [](const Tensor& t) { return t.log(); }, 0.1, 20.0, 1e-2, true},
        {"exp", [](const Tensor& t) { return t.exp(); }, -20.0, 2.0, 0.1, true},
        {"relu_positive", [](const Tensor& t) { return t.relu(); }, 0.2, 20.0, 1e-3, true},
        {"relu_negative", [](const Tensor& t) { return t.relu(); }, -20.0, -0.2, 1e-3, false},
        {"abs_positive", [](const Tensor& t) { return t.abs(); }, 0.2, 20.0, 1e-3, true},
        {"abs_negative", [](const Tensor& t) { return t.abs(); }, -20.0, -0.2, 1e-3, true},
        {"rsqrt", [](const Tensor& t) { return t.rsqrt(); }, 0.5, 5.0, 1e-3, true},
    };
    for (const Case& c : cases) {
        auto fn = c.fn;
        Tensor A = uniform(c.lo, c.hi, {2, 3, 4});
        gradient_same(c.name, [fn](vector<Tensor>& xs) { return fn(xs[0]); }, {A}, c.tol, 1e-4, c.nonzero);
    }
}

// dali/tensor/op/binary_tests.cpp:15-25, 57-92: one evaluation per forward op; add / subtract / eltmul / eltdiv / pow
static void binary_gradients() {
    utils::random::set_seed(101);
    {
        Tensor a({2, 3}, DTYPE_FLOAT), b({2, 3}, DTYPE_FLOAT);
        a.w = 2.0;
        b.w = 3.0;
        Tensor c = a + b;
        CHECK(std::fabs((double)Array(c.w.sum()) - 30.0) < 1e-6);
        graph::clear();
    }
    Tensor A = uniform(-2.0, 2.0, {3, 4}), B = uniform(0.5, 2.0, {3, 4});
    gradient_same("add", [](vector<Tensor>& xs) { return xs[0] + xs[1]; }, {A, B}, 1e-5);
    gradient_same("subtract", [](vector<Tensor>& xs) { return xs[0] - xs[1]; }, {A, B}, 1e-5);
    gradient_same("eltmul", [](vector<Tensor>& xs) { return xs[0] * xs[1]; }, {A, B}, 1e-5);
    gradient_same("eltdiv", [](vector<Tensor>& xs) { return xs[0] / xs[1]; }, {A, B}, 1e-4);
    gradient_same("pow", [](vector<Tensor>& xs) { return xs[1] ^ xs[0]; }, {A, B}, 1e-4);
    {
        // Tensor (op) number wraps the number in a 0-dimensional Tensor; forward values only: the reference's
        // backward pass adds a 2-D gradient into that 0-dimensional one and asserts (assignment.cpp:120-123)
        graph::NoBackprop nb;
        Tensor s = (A * 2.0 + 1.0) / 4.0 - A;
        CHECK(std::fabs((double)Array(s.w.sum()) - (12 * 0.25 - 0.5 * (double)Array(A.w.sum()))) < 1e-9);
    }
    // binary_tests.cpp:94-102 add_recursive: a tensor used on both sides
    gradient_same("add_recursive", [](vector<Tensor>& xs) { return xs[0] + xs[0] * xs[0]; }, {A}, 1e-4);
    gradient_same("add many", [](vector<Tensor>& xs) { return tensor_ops::add({xs[0], xs[1], xs[0], xs[1]}); }, {A, B}, 1e-5);
    // a row added to every row of a matrix: the gradient of the row is reduced over the broadcast dim
    Tensor row = uniform(-1.0, 1.0, {4})[Broadcast()];
    gradient_same("add broadcast", [](vector<Tensor>& xs) { return (xs[0] + xs[1]).tanh(); }, {A, row}, 1e-5);
}

// dali/tensor/tests.cpp:24-82, 296-336: reductions over everything (values and gradients); :84-142 reductions over one
// axis: forward values only -- their backward passes are commented out in the reference (op/reducers.cpp:66-110),
// which is why the reference disables those tests
static void reduction_gradients() {
    utils::random::set_seed(102);
    Tensor M = uniform(-2.0, 2.0, {4, 5}), P = uniform(0.1, 2.0, {4, 5});
    // Tensor::sum() / mean(): the backward pass adds a [1, 1] gradient into a [4, 5] one with <<=, which the
    // reference refuses (assignment.cpp:126-133); the same std::runtime_error comes out of this back end
    for (int which = 0; which < 2; ++which) {
        graph::clear();
        Tensor s = which == 0 ? M.sum() : M.mean();
        s.grad();
        bool refused = false;
        try { graph::backward(); M.dw.eval(); } catch (const std::runtime_error& e) {
            refused = std::string(e.what()).find("Could not autoreduce_assign") != std::string::npos;
        }
        CHECK(refused);
        graph::clear();
        M.dw = Array::zeros_like(M.w);
    }
    gradient_same("L2_norm", [](vector<Tensor>& xs) { return xs[0].L2_norm(); }, {P}, 1e-4);
    gradient_same("max", [](vector<Tensor>& xs) { return xs[0].max(); }, {P}, 1e-4);
    gradient_same("min", [](vector<Tensor>& xs) { return xs[0].min(); }, {P}, 1e-4);
    // tests.cpp:24-32 sum_test, :296-336 mean / max / min known answers
    graph::NoBackprop nb;
    Tensor known({3, 4}, DTYPE_FLOAT);
    known.w = op::arange(12).reshape({3, 4}).astype(DTYPE_FLOAT);
    CHECK((double)Array(known.sum().w) == 66.0);
    CHECK((double)Array(known.mean().w) == 5.5);
    CHECK((double)Array(known.max().w) == 11.0 && (double)Array(known.min().w) == 0.0);
    CHECK((int)Array(known.argmax().w) == 11 && (int)Array(known.argmin().w) == 0);
    const vector<int> shape = {2, 3, 1, 1, 2, 3};
    Tensor A({2, 3, 1, 1, 2, 3}, DTYPE_FLOAT);
    A.w = op::arange(36).reshape(shape).astype(DTYPE_FLOAT);
    for (int axis = -6; axis < 6; ++axis) {
        const int ax = axis < 0 ? axis + 6 : axis;
        Tensor s = tensor_ops::sum(A, {axis}), m = tensor_ops::mean(A, {axis}), hi = tensor_ops::max(A, {axis}), lo = tensor_ops::min(A, {axis});
        CHECK(s.ndim() == 5 && (double)Array(s.w.sum()) == 630.0);
        CHECK(std::fabs((double)Array(m.w.sum()) * shape[ax] - 630.0) < 1e-3);
        CHECK((double)Array(hi.w.max()) == 35.0 && (double)Array(lo.w.min()) == 0.0);
        Tensor am = tensor_ops::argmax(A, axis);
        CHECK((int)Array(am.w.max()) == shape[ax] - 1);
    }
    Tensor kd = tensor_ops::sum(A, {1, 5}, true);
    CHECK(kd.shape() == vector<int>({2, 1, 1, 1, 2, 1}));
}

// dali/tensor/op/dot_tests.cpp:15-58, composite_tests.cpp:16-115
static void dot_gradients() {
    utils::random::set_seed(103);
    Tensor A = uniform(-2.0, 2.0, {4, 5}), B = uniform(-2.0, 2.0, {5, 3});
    gradient_same("dot_2D", [](vector<Tensor>& xs) { return tensor_ops::dot(xs[0], xs[1]); }, {A, B}, 1e-4);
    Tensor u = uniform(-2.0, 2.0, {6}), v = uniform(-2.0, 2.0, {4});
    gradient_same("outer", [](vector<Tensor>& xs) { return tensor_ops::outer(xs[0], xs[1]); }, {u, v}, 1e-4);
    Tensor u2 = uniform(-2.0, 2.0, {6});
    gradient_same("inner", [](vector<Tensor>& xs) { return tensor_ops::inner(xs[0], xs[1]); }, {u, u2}, 1e-4);
    gradient_same("matrix_vector_dot", [](vector<Tensor>& xs) { return tensor_ops::matrix_vector_dot(xs[0], xs[1]); },
                  {A, uniform(-2.0, 2.0, {5})}, 1e-4);
    gradient_same("dot of transposes", [](vector<Tensor>& xs) { return tensor_ops::dot(xs[1].transpose(), xs[0].transpose()); },
                  {A, B}, 1e-4);
    Tensor S = uniform(-2.0, 2.0, {4, 4});
    gradient_same("self_dot", [](vector<Tensor>& xs) { return tensor_ops::dot(xs[0], xs[0]); }, {S}, 1e-4);
    Tensor T3 = uniform(-1.0, 1.0, {2, 3, 4}), T3b = uniform(-1.0, 1.0, {4, 3, 2});
    gradient_same("tensordot", [](vector<Tensor>& xs) { return tensor_ops::tensordot(xs[0], xs[1], {1, 2}, {1, 0}); }, {T3, T3b}, 1e-4);
    {
        // tensordot goes through dimshuffle + reshape of its operands (tensordot_as_dot.h): its values against loops
        graph::NoBackprop nb;
        Tensor td = tensor_ops::tensordot(T3, T3b, {1, 2}, {1, 0});
        vector<double> a = to_host(T3.w), b = to_host(T3b.w), got = to_host(td.w);
        CHECK(td.shape() == vector<int>({2, 2}));
        double worst = 0.0;
        for (int i = 0; i < 2; ++i)
            for (int l = 0; l < 2; ++l) {
                double want = 0.0;
                for (int j = 0; j < 3; ++j)
                    for (int k = 0; k < 4; ++k) want += a[(i * 3 + j) * 4 + k] * b[(k * 3 + j) * 2 + l];
                worst = std::max(worst, std::fabs(want - got[i * 2 + l]));
            }
        CHECK(worst < 1e-12);
    }

    const int num_examples = 20, hidden_size = 10, input_size = 5, other_input_size = 7;
    Tensor X = uniform(-10, 10, {num_examples, input_size}), W = uniform(-10, 10, {input_size, hidden_size});
    Tensor X2 = uniform(-10, 10, {num_examples, other_input_size}), W2 = uniform(-10, 10, {other_input_size, hidden_size});
    Tensor bias = uniform(-2, 2, {hidden_size})[Broadcast()];
    gradient_same("dot_with_bias", [](vector<Tensor>& xs) { return tensor_ops::dot_with_bias(xs[0], xs[1], xs[2]); }, {X, W, bias}, 1e-4);
    gradient_same("multiple_dot_with_bias",
                  [](vector<Tensor>& xs) { return tensor_ops::multiple_dot_with_bias({xs[0], xs[2]}, {xs[1], xs[3]}, xs[4]); },
                  {X, W, X2, W2, bias}, 3e-4);
    Tensor L = uniform(-2.0, 2.0, {2, 4}), Mid = uniform(-2.0, 2.0, {2, 3}), R = uniform(-2.0, 2.0, {3, 5});
    gradient_same("quadratic_form", [](vector<Tensor>& xs) { return tensor_ops::quadratic_form(xs[0], xs[1], xs[2]); }, {L, Mid, R}, 1e-4);
}

// dali/tensor/tests.cpp:266-294: views of a Tensor share w and dw with their parent (values checked here; a
// gradient that a backward pass adds into such a temporary view handle is a pending lazy assignment that dies with
// the handle, in the reference as here, so no gradient is expected through them); :450-482 hstack / vstack /
// concatenate and op/reshape_tests.cpp gather carry gradients
static void views_and_reshapes() {
    utils::random::set_seed(104);
    Tensor A = uniform(-2.0, 2.0, {4, 6}), B = uniform(-2.0, 2.0, {4, 3});
    {
        graph::NoBackprop nb;
        A.w.eval();
        vector<double> a = to_host(A.w);
        Tensor rows = A[Slice(1, 3)], cols = A.pluck_axis(1, Slice(3, 6)), At = A.transpose(), R = A.reshape({3, 8});
        CHECK(rows.shape() == vector<int>({2, 6}) && cols.shape() == vector<int>({4, 3}));
        CHECK(At.shape() == vector<int>({6, 4}) && R.shape() == vector<int>({3, 8}) && A.ravel().shape() == vector<int>({24}));
        CHECK(std::fabs((double)Array(rows.w[1][2]) - a[2 * 6 + 2]) < 1e-12);
        CHECK(std::fabs((double)Array(cols.w[3][1]) - a[3 * 6 + 4]) < 1e-12);
        CHECK(std::fabs((double)Array(At.w[5][2]) - a[2 * 6 + 5]) < 1e-12);
        CHECK(std::fabs((double)Array(R.w[2][7]) - a[23]) < 1e-12);
        // a write through the view's dw lands in the parent's dw
        rows.dw += 2.0;
        rows.dw.eval();
        CHECK(std::fabs((double)Array(A.dw.sum()) - 24.0) < 1e-12);
        A.dw.clear();
    }
    // gradients through views: the backward pass adds into a temporary handle on a view of the parent's dw; the update
    // runs when it is written on this back end, so it lands (in the reference it stays pending in that handle and is
    // lost with it, which is why the reference disables these tests)
    gradient_same("slice", [](vector<Tensor>& xs) { return Tensor(xs[0][Slice(1, 3)]).tanh(); }, {A}, 1e-4);
    gradient_same("column slices", [](vector<Tensor>& xs) {
        return xs[0].pluck_axis(1, Slice(0, 3)) * xs[0].pluck_axis(1, Slice(3, 6)); }, {A}, 1e-4);
    gradient_same("transpose", [](vector<Tensor>& xs) { return tensor_ops::dot(xs[0].transpose(), xs[0]); }, {A}, 1e-4);
    gradient_same("reshape", [](vector<Tensor>& xs) { return xs[0].reshape({3, 8}).square(); }, {A}, 1e-4);
    gradient_same("ravel", [](vector<Tensor>& xs) { return xs[0].ravel().sigmoid(); }, {A}, 1e-4);
    gradient_same("hstack", [](vector<Tensor>& xs) { return tensor_ops::hstack({xs[0], xs[1]}).square(); }, {A, B}, 1e-4);
    Tensor C = uniform(-2.0, 2.0, {2, 6});
    gradient_same("vstack", [](vector<Tensor>& xs) { return tensor_ops::vstack({xs[0], xs[1]}).tanh(); }, {A, C}, 1e-4);
    gradient_same("concatenate", [](vector<Tensor>& xs) { return tensor_ops::concatenate({xs[0], xs[1], xs[0]}, 1).exp(); }, {A, B}, 1e-3);
    // rows of an embedding matrix picked by index; repeated indices accumulate in the gradient
    Tensor E = uniform(-2.0, 2.0, {5, 3});
    Tensor idx({4}, DTYPE_INT32);
    idx.w = op::arange(4);
    idx.w(3).assign(1).eval();
    idx.constant = true;
    gradient_same("gather", [idx](vector<Tensor>& xs) { return tensor_ops::gather(xs[0], idx).square(); }, {E}, 1e-4);
    gradient_same("index tensor", [idx](vector<Tensor>& xs) { return xs[0][idx].tanh(); }, {E}, 1e-4);
}

// an LSTM cell written with the tensor layer the way dali/layers/lstm.cpp:82-87, 226-263 builds it: one stacked
// input layer (x Wx + h Wh + b) per gate, then c' = f c + i g, h' = o tanh(c').  p = {x, h, c, then per gate Wx, Wh, b}
static Tensor lstm_cell(vector<Tensor>& p) {
    auto gate = [&p](int k) { return tensor_ops::multiple_dot_with_bias({p[0], p[1]}, {p[3 + 3 * k], p[4 + 3 * k]}, p[5 + 3 * k]); };
    Tensor i = gate(0).sigmoid(), f = gate(1).sigmoid(), o = gate(2).sigmoid(), g = gate(3).tanh();
    Tensor c_new = f * p[2] + i * g;
    return o * c_new.tanh();
}

// the same cell with one [H, 4H] weight matrix per input and the gates as column slices of one product (the
// benchmark's layout): gradients flow through the slices
static Tensor lstm_cell_sliced(vector<Tensor>& p, int H) {
    Tensor gates = tensor_ops::multiple_dot_with_bias({p[0], p[1]}, {p[3], p[4]}, p[5]);
    Tensor i = gates.pluck_axis(1, Slice(0, H)).sigmoid(), f = gates.pluck_axis(1, Slice(H, 2 * H)).sigmoid();
    Tensor o = gates.pluck_axis(1, Slice(2 * H, 3 * H)).sigmoid(), g = gates.pluck_axis(1, Slice(3 * H, 4 * H)).tanh();
    Tensor c_new = f * p[2] + i * g;
    return o * c_new.tanh();
}

static void lstm_cell_gradients() {
    utils::random::set_seed(105);
    {
        const int B = 3, H = 4;
        vector<Tensor> p = {uniform(-1, 1, {B, H}), uniform(-1, 1, {B, H}), uniform(-1, 1, {B, H}), uniform(-0.5, 0.5, {H, 4 * H}),
                            uniform(-0.5, 0.5, {H, 4 * H}), uniform(-0.5, 0.5, {4 * H})[Broadcast()]};
        gradient_same("lstm cell, sliced gates", [H](vector<Tensor>& xs) { return lstm_cell_sliced(xs, H); }, p, 1e-4);
    }
    const int B = 3, H = 4;
    vector<Tensor> p = {uniform(-1, 1, {B, H}), uniform(-1, 1, {B, H}), uniform(-1, 1, {B, H})};
    for (int k = 0; k < 4; ++k) {
        p.push_back(uniform(-0.5, 0.5, {H, H}));
        p.push_back(uniform(-0.5, 0.5, {H, H}));
        p.push_back(uniform(-0.5, 0.5, {H})[Broadcast()]);
    }
    gradient_same("lstm cell", [](vector<Tensor>& xs) { return lstm_cell(xs); }, p, 1e-4);
    // the benchmark's size in fp32: one forward and backward pass, every gradient finite and not all zero
    const int BB = 256, HH = 1024;
    auto f32 = [](double lo, double hi, const vector<int>& s) { return Tensor::uniform(Array((float)lo), Array((float)hi), s); };
    vector<Tensor> q = {f32(-1, 1, {BB, HH}), f32(-1, 1, {BB, HH}), f32(-1, 1, {BB, HH})};
    for (int k = 0; k < 4; ++k) {
        q.push_back(f32(-0.03, 0.03, {HH, HH}));
        q.push_back(f32(-0.03, 0.03, {HH, HH}));
        q.push_back(f32(-0.1, 0.1, {HH})[Broadcast()]);
    }
    graph::clear();
    Tensor hn = lstm_cell(q);
    hn.grad();
    graph::backward();
    for (Tensor& t : q) {
        t.dw.eval();
        CHECK(!t.is_grad_nan());
        CHECK((double)Array(op::sum(op::abs(t.dw))) > 0.0);
    }
    CHECK(hn.w.shape() == vector<int>({BB, HH}) && !hn.is_nan());
    // wall time of a forward + backward step (host lowering included), for the record
    const int steps = 10;
    double ms = 0.0;
    for (int it = 0; it < steps + 2; ++it) {
        for (Tensor& t : q) t.dw.clear();
        for (Tensor& t : q) t.dw.eval();
        (void)(double)Array(q[0].dw.sum());
        auto t0 = std::chrono::steady_clock::now();
        graph::clear();
        Tensor h2 = lstm_cell(q);
        h2.grad();
        graph::backward();
        vector<Array> grads;
        for (Tensor& t : q) grads.push_back(t.dw);
        for (Array& g : grads) g.eval(false);
        (void)(double)Array(q[3].dw(0));
        auto t1 = std::chrono::steady_clock::now();
        if (it >= 2) ms += std::chrono::duration<double, std::milli>(t1 - t0).count();
    }
    std::printf("lstm cell forward + backward at [256, 1024], fp32, through the reference's tape: %.3f ms per step\n", ms / steps);
}

// dali/tensor/tape.h:28-43 NoBackprop; consider_constant; dali/tensor/tests.cpp:904-911 trivial_sgd restated by hand
static void tape_and_training() {
    utils::random::set_seed(106);
    Tensor A = uniform(-1, 1, {3, 3});
    graph::clear();
    {
        graph::NoBackprop nb;
        Tensor B = A.tanh() * A;
        (void)B;
        CHECK(graph::size() == 0);
    }
    Tensor B = A.tanh() * A;
    CHECK(graph::size() == 2);
    graph::clear();
    Tensor Cc = tensor_ops::consider_constant(A);
    Tensor D = Cc * Cc;
    D.grad();
    graph::backward();
    CHECK((double)Array(op::sum(op::abs(A.dw))) == 0.0);

    // least squares by gradient descent: y = X W*, W learned from zero
    const int n = 64, d = 8;
    Tensor X = uniform(-1, 1, {n, d}), W_true = uniform(-1, 1, {d, 1});
    X.constant = true;
    Tensor y(op::dot(X.w, W_true.w), true);
    y.constant = true;
    Tensor W({d, 1}, DTYPE_DOUBLE);
    double first = 0.0, last = 0.0;
    for (int step = 0; step < 200; ++step) {
        Tensor err = (tensor_ops::dot(X, W) - y).square();      // objective = sum of the entries (Tensor::grad)
        err.grad();
        graph::backward();
        const double e = (double)Array(err.w.sum()) / n;
        if (step == 0) first = e;
        last = e;
        W.w -= W.dw * (0.5 / n);
        W.w.eval();
        W.dw.clear();
    }
    CHECK(first > 0.05);
    CHECK(last < 1e-6 * first);
    CHECK((int)Array(op::all_close(W.w, W_true.w, 1e-3)) != 0);
}

// dali/tensor/tests.cpp:876-955 test_solver_trivial: every solver of dali/tensor/solver.cpp drives the norm of a
// five-element vector below 0.1 within 200 steps (the reference's step sizes)
static void solvers() {
    typedef std::function<std::shared_ptr<solver::AbstractSolver>(vector<Tensor>)> create_solver_t;
    struct Case { const char* name; create_solver_t create; };
    const vector<Case> cases = {
        {"sgd", [](vector<Tensor> p) { auto s = std::make_shared<solver::SGD>(p); s->step_size = 0.3; s->clip_norm = 0; return s; }},
        {"adagrad", [](vector<Tensor> p) { auto s = std::make_shared<solver::AdaGrad>(p); s->step_size = 1; s->clip_norm = 0.0; return s; }},
        {"rmsprop", [](vector<Tensor> p) { auto s = std::make_shared<solver::RMSProp>(p); s->step_size = 0.1; s->clip_norm = 0.0; return s; }},
        {"rmspropmomentum", [](vector<Tensor> p) { auto s = std::make_shared<solver::RMSPropMomentum>(p); s->step_size = 0.5; s->momentum = 0.2; return s; }},
        {"adadelta", [](vector<Tensor> p) { auto s = std::make_shared<solver::AdaDelta>(p); s->clip_norm = 0.0; s->rho = 0.1; return s; }},
        {"adam", [](vector<Tensor> p) { auto s = std::make_shared<solver::Adam>(p); s->step_size = 0.005; return s; }},
    };
    const double initial[5] = {8.98117318, 1.38778046, -2.56764083, 7.99331316, 0.0};
    for (const Case& c : cases) {
        ++checks;
        try {
            graph::clear();
            Tensor X({5}, DTYPE_DOUBLE);
            for (int i = 0; i < 5; ++i) X.w(i).assign(initial[i]).eval();
            vector<Tensor> params({X});
            auto solver = c.create(params);
            double last_error = (double)Array(X.L2_norm().w);
            bool started_high = last_error > 10.0;
            graph::clear();
            int iter = 0;
            for (; iter < 200 && last_error >= 0.1; ++iter) {
                Tensor error = X.L2_norm();
                error.grad();
                graph::backward();
                solver->step(params);
                last_error = (double)Array(error.w);
            }
            const bool ok = started_high && last_error < 0.1;
            std::printf("case solver %s: %s (norm %.4g after %d steps)\n", c.name, ok ? "ok" : "wrong", last_error, iter);
            if (!ok) ++failures;
        } catch (const std::runtime_error& e) {
            graph::clear();
            std::printf("case solver %s: throws\n  (%s)\n", c.name, e.what());
            ++thrown;
        }
    }
}

// dali/tensor/tests.cpp:225-241 TensorIOTests.save_load_test
static void save_and_load(const std::string& dir) {
    Tensor A = uniform(-2, 2, {3, 5});
    A.w.eval();
    Tensor::save(dir + "/tensor_smoke.npy", A);
    Tensor loaded = Tensor::load(dir + "/tensor_smoke.npy");
    CHECK(loaded.shape() == A.shape() && loaded.dtype() == DTYPE_DOUBLE);
    CHECK(tensor_ops::equals(A, loaded));
}

static void section(const char* name, const std::function<void()>& body) {
    try {
        body();
    } catch (const std::exception& e) {
        graph::clear();
        std::printf("section %s: throws\n  (%s)\n", name, e.what());
        ++failures;
    }
}

int main(int argc, char** argv) {
    const std::string dir = argc > 1 ? argv[1] : "/tmp";
    std::setvbuf(stdout, nullptr, _IOLBF, 0);
    section("unary", unary_gradients);
    section("binary", binary_gradients);
    section("reductions", reduction_gradients);
    section("dot", dot_gradients);
    section("views", views_and_reshapes);
    section("lstm", lstm_cell_gradients);
    section("tape", tape_and_training);
    section("solvers", solvers);
    section("io", [&dir]() { save_and_load(dir); });
    std::printf("{\"checks\": %d, \"failures\": %d, \"throws\": %d}\n", checks, failures, thrown);
    return failures == 0 ? 0 : 1;
}
