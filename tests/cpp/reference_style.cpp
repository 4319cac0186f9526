// Written the way a user of the reference writes code: its include paths, class Array, namespace
// op::, lazy expressions, implicit evaluation on scalar conversion -- compiled against the C++
// headers of this back end and linked with libdali_b200.so.  Each block restates, in this file's
// own words, what a test of the reference's suite asserts (file:line given), so that "existing
// code keeps working" is checked through the C++ API itself and not only through the C binding.
// Needs a GPU (built on any machine by __graft_entry__.build(), run by tests/test_gpu_cpp_api.py).
#include <cmath>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "dali/array/array.h"
#include "dali/array/op.h"
#include "dali/array/op/arange.h"
#include "dali/array/op/eye.h"
#include "dali/array/op/one_hot.h"
#include "dali/array/op/outer.h"
#include "dali/array/op/scan.h"
#include "dali/array/op/softmax.h"
#include "dali/array/expression/computation.h"
#include "dali/array/expression/expression.h"
#include "dali/array/expression/optimization.h"
#include "dali/utils/random.h"
#include "dali/utils/scope.h"

static int checks = 0, failures = 0;
#define CHECK(cond)                                                                   \
    do {                                                                              \
        ++checks;                                                                     \
        if (!(cond)) { ++failures; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)
#define CHECK_NEAR(a, b, tol) CHECK(std::fabs((double)(a) - (double)(b)) <= (tol))
#define CHECK_THROWS(stmt)                                                            \
    do {                                                                              \
        ++checks;                                                                     \
        bool thrown = false;                                                          \
        try { stmt; } catch (const std::runtime_error&) { thrown = true; }            \
        if (!thrown) { ++failures; std::printf("FAILED %s:%d: no std::runtime_error from %s\n", __FILE__, __LINE__, #stmt); } \
    } while (0)

// dali/array/tests/tests.cpp:166-214: in-place operators with a reshaped arange on the right
static void inplace_with_arange() {
    Array x = Array::zeros({3, 2}, DTYPE_INT32);
    x = 10;
    x += op::arange(6).reshape({3, 2});
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 2; ++j) CHECK((int)x[i][j] == 10 + i * 2 + j);
    x -= op::arange(6).reshape({3, 2});
    x *= op::arange(6).reshape({3, 2});
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 2; ++j) CHECK((int)x[i][j] == 10 * (i * 2 + j));
}

// tests.cpp:245-277: a diagonal assigned into an int matrix, another one subtracted
static void eye_init() {
    Array myeye({4, 5}, DTYPE_INT32);
    const double diag = 5.0;
    myeye.assign(op::diag(diag, 4, 5));
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 5; ++j) CHECK((int)myeye[i][j] == (i == j ? 5 : 0));
    myeye -= op::diag(1.0, 4, 5);
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 5; ++j) CHECK((int)myeye[i][j] == (i == j ? 4 : 0));
}

// tests.cpp:1120-1164: reducers and arg-reducers, known answers
static void reducers() {
    Array a = op::arange(50).reshape({5, 10}).astype(DTYPE_FLOAT);
    CHECK((int)a.sum() == 50 * 49 / 2);
    Array p = op::arange(1, 6);
    CHECK((int)op::prod(p) == 120);
    Array r = op::arange(-100, 42);
    CHECK((int)r.max() == 41 && (int)r.min() == -100);
    CHECK((int)r.argmax() == 141 && (int)r.argmin() == 0);
    Array m = op::arange(20).reshape({4, 5});
    Array am0 = op::argmax(m, 0), am1 = op::argmax(m, 1);
    for (int j = 0; j < 5; ++j) CHECK((int)am0[j] == 3);
    for (int i = 0; i < 4; ++i) CHECK((int)am1[i] == 4);
    Array ones = Array::ones({2, 3, 4, 5}, DTYPE_INT32);
    Array s = op::sum(ones, {-1});
    CHECK(s.shape() == std::vector<int>({2, 3, 4}) && (int)s[1][2][3] == 5);
}

// tests.cpp:1622-1664: the spelled-out softmax is one fused kernel and equals op::softmax; rows sum to 1
static void fused_softmax() {
    utils::random::set_seed(1234);
    Array a = op::uniform(Array(-20.0f), Array(20.0f), {5, 10});
    a.eval();
    Array exped = op::exp(a - op::max(a, {-1}, true));
    Array fused = exped / op::sum(exped, {-1}, true);
    Array lib = op::softmax(a, -1);
    CHECK(Array::allclose(fused, lib, 1e-6));
    Array rows = op::sum(fused, {-1});
    for (int i = 0; i < 5; ++i) CHECK_NEAR((float)rows[i], 1.0, 1e-5);
}

// tests.cpp:1266-1361: gather, gather_from_rows and scatter-add through a gathered view
static void gather_scatter() {
    Array source = op::arange(5 * 6).reshape({5, 6});
    Array indices = Array::zeros({3}, DTYPE_INT32);
    // an element assignment is lazy like every other: it runs when evaluated (tests.cpp:994, 1288)
    (indices[0] = 4).eval(); (indices[1] = 0).eval(); (indices[2] = 4).eval();
    Array g = source[indices];
    CHECK(g.shape() == std::vector<int>({3, 6}));
    CHECK((int)g[0][2] == 26 && (int)g[1][5] == 5 && (int)g[2][0] == 24);
    Array rows = op::gather_from_rows(source, op::arange(5));
    for (int i = 0; i < 5; ++i) CHECK((int)rows[i] == i * 6 + i);
    Array dest = Array::zeros({3}, DTYPE_INT32);
    Array idx = Array::zeros({6}, DTYPE_INT32);
    int where[6] = {0, 0, 1, 1, 1, 2};
    for (int k = 0; k < 6; ++k) (idx[k] = where[k]).eval();
    Array gathered = dest[idx];
    gathered += 1;
    gathered.eval();
    CHECK((int)dest[0] == 2 && (int)dest[1] == 3 && (int)dest[2] == 1);
}

// dali/array/tests/dot_tests.cpp:37-67: small integer products, all operand layouts
static void dot_known_answers() {
    Array a = op::arange(6).reshape({2, 3}).astype(DTYPE_FLOAT);
    Array b = op::arange(12).reshape({3, 4}).astype(DTYPE_FLOAT);
    Array c = op::dot(a, b);
    const int want[2][4] = {{20, 23, 26, 29}, {56, 68, 80, 92}};
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 4; ++j) CHECK((int)c[i][j] == want[i][j]);
    Array ct = op::dot(b.transpose(), a.transpose());      // (a.b)^T through transposed views
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 4; ++j) CHECK((int)ct[j][i] == want[i][j]);
    CHECK_THROWS(op::dot(a, a).eval());                      // dot_tests.cpp:213-216
}

// tests.cpp:985-1012: one_hot against an element-by-element construction
static void one_hot() {
    Array idx = op::uniform(Array(0), Array(6), {2, 3});
    idx.eval();
    Array oh = op::one_hot(idx, 7, 112.2, 42.0);
    CHECK(oh.dtype() == DTYPE_DOUBLE && oh.shape() == std::vector<int>({2, 3, 7}));
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 3; ++j)
            for (int d = 0; d < 7; ++d) CHECK((double)oh[i][j][d] == ((int)idx[i][j] == d ? 112.2 : 42.0));
}

// tests.cpp:968-983 and 1737-1771: outer products of lazy operands; running sums and products
static void outer_and_scans() {
    Array x = op::arange(3).astype(DTYPE_FLOAT), y = op::arange(4).astype(DTYPE_FLOAT);
    Array o = op::outer(op::tanh(x - 3.0f), op::tanh(y - 2.0f));
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 4; ++j) CHECK_NEAR((float)o[i][j], std::tanh(i - 3.0) * std::tanh(j - 2.0), 1e-5);
    Array a = op::arange(0, 20);
    Array inc = op::cumsum(a, true), exc = op::cumsum(a.reshape({2, 10}), false);
    CHECK(exc.shape() == std::vector<int>({2, 11}));
    int run = 0;
    for (int i = 0; i < 20; ++i) { run += i; CHECK((int)inc[i] == run); }
    CHECK((int)exc[1][0] == 0 && (int)exc[1][1] == 10 && (int)exc[1][10] == 145);
    Array p = op::cumprod(op::arange(1, 11), true);
    CHECK((int)p[9] == 3628800);
}

// Benchmark configuration 2 in miniature: the LSTM cell written with op::, against plain loops
static void lstm_cell() {
    const int B = 4, H = 8;
    utils::random::set_seed(7);
    Array x = op::normal(Array(0.0f), Array(1.0f), {B, H}), h = op::normal(Array(0.0f), Array(1.0f), {B, H});
    Array c = op::normal(Array(0.0f), Array(1.0f), {B, H});
    Array Wx = op::normal(Array(0.0f), Array(0.3f), {H, 4 * H}), Wh = op::normal(Array(0.0f), Array(0.3f), {H, 4 * H});
    Array b = op::normal(Array(0.0f), Array(0.1f), {4 * H});
    for (Array* t : {&x, &h, &c, &Wx, &Wh, &b}) t->eval();
    Array gates = op::dot(x, Wx) + op::dot(h, Wh) + b[Broadcast()];
    Array i = op::sigmoid(gates[Slice()][Slice(0, H)]), f = op::sigmoid(gates[Slice()][Slice(H, 2 * H)]);
    Array o = op::sigmoid(gates[Slice()][Slice(2 * H, 3 * H)]), g = op::tanh(gates[Slice()][Slice(3 * H, 4 * H)]);
    Array c_new = f * c + i * g;
    Array h_new = o * op::tanh(c_new);
    auto sig = [](double v) { return 1.0 / (1.0 + std::exp(-v)); };
    for (int r = 0; r < B; ++r)
        for (int k = 0; k < H; ++k) {
            double pre[4];
            for (int q = 0; q < 4; ++q) {
                double s = (float)b[q * H + k];
                for (int t = 0; t < H; ++t) s += (double)(float)x[r][t] * (float)Wx[t][q * H + k] + (double)(float)h[r][t] * (float)Wh[t][q * H + k];
                pre[q] = s;
            }
            const double cn = sig(pre[1]) * (float)c[r][k] + sig(pre[0]) * std::tanh(pre[3]);
            CHECK_NEAR((float)c_new[r][k], cn, 1e-5);
            CHECK_NEAR((float)h_new[r][k], sig(pre[2]) * std::tanh(cn), 1e-5);
        }
}

// tests.cpp:372-468, 470-550: views of a [2,3,4] arange: shapes, offsets, strides, sums, in-place update of a strided view
static Array build_234_arange() { return op::arange(24).reshape({2, 3, 4}); }
static void views_of_an_arange() {
    Array x = build_234_arange();
    CHECK(x.contiguous_memory());
    Array p0 = x.pluck_axis(0, 1);
    CHECK(p0.shape() == std::vector<int>({3, 4}) && p0.number_of_elements() == 12 && p0.offset() == 12 && p0.strides().empty());
    Array p1 = x.pluck_axis(1, 2);
    CHECK(p1.shape() == std::vector<int>({2, 4}) && p1.offset() == 8 && p1.strides() == std::vector<int>({12, 1}));
    Array p2 = x.pluck_axis(2, 1);
    CHECK(p2.shape() == std::vector<int>({2, 3}) && p2.offset() == 1 && p2.strides() == std::vector<int>({12, 4}));
    CHECK(x.memory().get() == p1.memory().get() && !p1.contiguous_memory());
    CHECK((int)x.pluck_axis(0, 0).sum() == 66);
    CHECK((int)p1.sum() == 8 + 9 + 10 + 11 + 20 + 21 + 22 + 23);
    CHECK((int)p2.sum() == 1 + 5 + 9 + 13 + 17 + 21);
    p2 += 1;                                                     // tests.cpp:517-530
    CHECK((int)p2.sum() == 6 + 1 + 5 + 9 + 13 + 17 + 21);
    CHECK((int)x[0][0][1] == 2 && (int)x[0][0][0] == 0);
    Array y = build_234_arange();
    Array sliced = y[Slice(0, -1)][2][Slice(0, 4, -2)];          // tests.cpp:548-553
    CHECK((int)sliced.sum() == 20);
    CHECK(Slice(0, 5).size() == 5 && Slice(0, 5, 2).size() == 3 && Slice(0, 5, -2).size() == 3 && Slice(0, 7, -3).size() == 3);
    CHECK(Slice(0, 12, 2).contains(0) && !Slice(0, 12, 2).contains(1) && !Slice(0, 12, -2).contains(0) && Slice(0, 12, -2).contains(1));
    CHECK_THROWS(Slice(0, 2, 0));
    Array r({2, 3, 4}, DTYPE_INT32);                              // tests.cpp:424-434
    CHECK(r.reshape({6, -1}).shape() == std::vector<int>({6, 4}) && r.reshape({-1, 2}).shape() == std::vector<int>({12, 2}));
    CHECK_THROWS(r.reshape({-1, -1}));
    CHECK_THROWS(r.reshape({-1, 5}));
}

// tests.cpp:555-585 in small: every (start, end, step) slice of every dim, sums against a host loop
static void double_striding() {
    Array x = op::uniform(Array(-1000), Array(1000), {2, 3, 4});
    x.eval();
    int host[24];
    for (int i = 0; i < 24; ++i) host[i] = (int)x(i);
    auto slices = [](int dim) {
        std::vector<Slice> out;
        for (int start = 0; start < dim; ++start)
            for (int end = start + 1; end <= dim; ++end)
                for (int step = -2; step < 3; ++step)
                    if (step != 0) out.push_back(Slice(start, end, step));
        return out;
    };
    int n = 0;
    for (auto& s0 : slices(2))
        for (auto& s1 : slices(3))
            for (auto& s2 : slices(4)) {
                if ((n++ % 7) != 0) continue;                     // every seventh combination: ~700 kernels otherwise
                Array sliced = x[s0][s1][s2];
                int want = 0;
                for (int i = 0; i < 2; ++i)
                    for (int j = 0; j < 3; ++j)
                        for (int k = 0; k < 4; ++k)
                            if (s0.contains(i) && s1.contains(j) && s2.contains(k)) want += host[i * 12 + j * 4 + k];
                CHECK((int)sliced.sum() == want);
            }
}

// tests.cpp:388-421: copies and references
static void copies() {
    Array original = op::arange(9).reshape({3, 3});
    Array copy(original, true);
    copy += 1;
    for (int i = 0; i < 9; ++i) CHECK((int)original(i) != (int)copy(i));
    Array original2 = op::arange(9).reshape({3, 3});
    Array view(original2, false);
    view += 2;
    for (int i = 0; i < 9; ++i) CHECK((int)original2(i) == (int)view(i));
}

// expression/control_flow.h:33: a result that must see a pending in-place update
static void control_dependency() {
    Array x = Array::zeros({4}, DTYPE_INT32);
    Array update = x;
    update += 3;                                   // lazy: nothing has run yet
    Array y = op::control_dependency(update, x) * 2;
    for (int i = 0; i < 4; ++i) CHECK((int)y[i] == 6);
}

// tests.cpp:124-125, 438-440, 613: shape and rank violations surface as std::runtime_error
static void errors() {
    Array a({3, 4}), b({4, 3});
    CHECK_THROWS(a + b);
    CHECK_THROWS(a.reshape({5, 5}));
    CHECK_THROWS(a[7]);
    CHECK_THROWS(op::one_hot(a, 3, 1.0, 0.0));
}

// dali/array/tests/dot_tests.cpp:10-35: a product of two evaluated operands runs exactly ONE computation, which a
// ScopeObserver sees as one scope being left; nothing runs before eval() is called
static void laziness_counted_by_scopes() {
    Array a = Array::ones({2, 3}, DTYPE_FLOAT);
    Array b = op::arange(12).reshape({4, 3}).astype(DTYPE_FLOAT);
    b = b.transpose();
    b.eval();
    a.eval();
    int computations = 0;
    std::vector<std::string> names;
    {
        auto cb = ScopeObserver(NULL, [&](const ScopeObserver::State& state) {
            computations += 1;
            names.push_back(*state.trace.back());
        });
        Array c = op::dot(a, b);
        CHECK(computations == 0);            // lazy: building the expression ran nothing
        c.eval();
        const float expected[] = {3, 12, 21, 30, 3, 12, 21, 30};
        for (int i = 0; i < c.number_of_elements(); ++i) CHECK((float)c(i) == expected[i]);
        CHECK(computations == 1);
        CHECK(names.size() == 1 && names[0].find("MatMul") == 0);
        // a fused softmax is one computation too (plus the compile-or-load step it contains)
        computations = 0;
        names.clear();
        Array x = op::arange(10).reshape({2, 5}).astype(DTYPE_FLOAT);
        x.eval();
        computations = 0;
        names.clear();
        Array s = op::softmax(x, -1);
        s.eval();
        int jit = 0;
        for (const std::string& n : names) jit += n == "get_function";
        CHECK(computations - jit == 1 && jit == 1);
    }
    CHECK(!Scope::has_observers());
}

// computation.h:20-38: an implementation registered for a node class is asked first and may decline
struct FillWithSeven : public Computation {
    using Computation::Computation;
    void run() override {
        float* out = (float*)left_data(memory::Device::cpu());
        for (int i = 0; i < left_.number_of_elements(); ++i) out[i] = 7.0f;
        (void)argument_data(memory::Device::cpu(), 0);       // the value's first argument, fresh on the host
    }
};
static bool g_claim_products = false;
static int g_factory_calls = 0;
static void plug_in_registry() {
    register_implementation(typeid(MatMul).name(), [](Array dest, OPERATOR_T op, Array x, Array assignment) -> std::shared_ptr<Computation> {
        ++g_factory_calls;
        if (!g_claim_products || dest.dtype() != DTYPE_FLOAT) return nullptr;        // decline: the built-in GEMM runs
        return std::make_shared<FillWithSeven>(dest, op, x, assignment);
    });
    Array a = Array::ones({4, 8}, DTYPE_FLOAT), b = Array::ones({8, 4}, DTYPE_FLOAT);
    Array c = op::dot(a, b);
    c.eval();
    CHECK(g_factory_calls == 1);
    CHECK((float)c[1][2] == 8.0f);
    g_claim_products = true;
    Array d = op::dot(a, b);
    d.eval();
    CHECK(g_factory_calls == 2);
    CHECK((float)d[1][2] == 7.0f && (float)d[3][3] == 7.0f);
    CHECK(d.is_buffer());
    g_claim_products = false;
    // the (name, predicate) form: only reductions to a scalar are claimed
    static int scalar_reductions = 0;
    register_implementation("count scalar reductions", [](const Array& v) { return as<Reduce>(v) != nullptr && v.ndim() == 0; },
                            [](Array, OPERATOR_T, Array, Array) -> std::shared_ptr<Computation> { ++scalar_reductions; return nullptr; });
    Array r = op::sum(a);
    CHECK((float)r == 32.0f);
    Array r2 = op::sum(a, {0});
    r2.eval();
    CHECK(scalar_reductions == 1);
}

// optimization.h:8-16: negate(negate(x)) is rewritten to x before anything is lowered
static void registered_optimization() {
    static int rewrites = 0;
    register_optimization(
        [](const Array& a) {
            Elementwise* outer = as<Elementwise>(a);
            if (!outer || outer->functor_ != "negate") return false;
            Elementwise* inner = as<Elementwise>(outer->arguments_[0]);
            return inner != nullptr && inner->functor_ == "negate";
        },
        [](const Array& a) { ++rewrites; return a.expression()->arguments_[0].expression()->arguments_[0]; }, "double negation");
    Array x = op::arange(6).reshape({2, 3}).astype(DTYPE_FLOAT);
    x.eval();
    Array y = -(-(x * 2.0f));
    Array z = canonical(y);
    CHECK(rewrites == 1);
    CHECK(z.is_assignment());
    CHECK(right_args(z).size() == 2);                 // eltmul(x, 2): the two negations are gone
    CHECK(z.expression_name() == "Assignment");
    y.eval();
    CHECK((float)y[1][2] == 10.0f);
}

int main() {
    try {
        laziness_counted_by_scopes();
        plug_in_registry();
        registered_optimization();
        inplace_with_arange();
        eye_init();
        reducers();
        fused_softmax();
        gather_scatter();
        dot_known_answers();
        one_hot();
        outer_and_scans();
        lstm_cell();
        control_dependency();
        views_of_an_arange();
        double_striding();
        copies();
        errors();
    } catch (const std::exception& e) {
        std::printf("EXCEPTION: %s\n", e.what());
        return 2;
    }
    std::printf("%s: %d checks, %d failures\n", failures ? "FAIL" : "PASS", checks, failures);
    return failures ? 1 : 0;
}
