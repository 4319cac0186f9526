// op:: free functions: build lazy expression nodes (reference:
// dali/array/op/{unary,binary,reducers,reducer_operation,elementwise_operation,
// gather,gather_from_rows,softmax,dot,arange}.cpp).
#include <algorithm>
#include <cmath>
#include <map>
#include <sstream>

#include "dali/array/op.h"
#include "dali/utils/random.h"
#include "dali/array/expression/expression.h"

static std::string shape_str(const std::vector<int>& s) {
    std::ostringstream o;
    o << "[";
    for (size_t i = 0; i < s.size(); ++i) o << (i ? ", " : "") << s[i];
    o << "]";
    return o.str();
}

namespace utils {
namespace random {
std::mt19937& generator() {
    static std::mt19937 gen(std::random_device{}());
    return gen;
}
void reseed() { generator().seed(std::random_device{}()); }
void set_seed(int new_seed) { generator().seed((unsigned)new_seed); }
}  // namespace random
int randint(int lower, int upper) { return std::uniform_int_distribution<int>(lower, upper)(random::generator()); }
double randdouble(double lower, double upper) { return std::uniform_real_distribution<double>(lower, upper)(random::generator()); }
}  // namespace utils

namespace op {

static std::string strip(const std::string& functor_name) {
    const std::string pre = "functor::";
    std::string n = functor_name.compare(0, pre.size(), pre) == 0 ? functor_name.substr(pre.size()) : functor_name;
    if (n == "isnotanumber" || n == "isinfinity") return n;
    return n;
}

// ---------------------------------------------------------------- elementwise
// bf16 is a storage type: whatever is computed on a bf16 Array is computed on its float values
static Array computed_in_float(const Array& a) { return a.dtype() == DTYPE_BF16 ? unsafe_cast(a, DTYPE_FLOAT) : a; }

Array elementwise(Array a, const std::string& functor_name) {
    DALI_ASSERT(!a.is_stateless(), "elementwise operation on a stateless Array");
    a = computed_in_float(a);
    return Array(std::make_shared<Elementwise>(strip(functor_name), std::vector<Array>({a}), a.shape(), a.dtype()));
}

// common shape of two same-rank operands: every dim equal or one of them 1
static std::vector<int> common_shape(const Array& a, const Array& b, const std::string& what) {
    if (a.ndim() == 0) return b.shape();
    if (b.ndim() == 0) return a.shape();
    std::vector<int> out(a.ndim());
    for (int d = 0; d < a.ndim(); ++d) {
        int x = a.shape()[d], y = b.shape()[d];
        DALI_ASSERT(x == y || x == 1 || y == 1,
                    "Arguments to binary operation '" + what + "' must have compatible shapes (got left.shape = " +
                        shape_str(a.shape()) + ", right.shape = " + shape_str(b.shape()) + ").");
        out[d] = x == 1 ? y : x;
    }
    return out;
}

std::tuple<Array, Array> ensure_arguments_compatible(Array a, Array b, const std::string& functor_name, bool update_shape) {
    DALI_ASSERT(!a.is_stateless() && !b.is_stateless(), "binary operation on a stateless Array");
    a = computed_in_float(a);
    b = computed_in_float(b);
    if (update_shape) {
        DALI_ASSERT(a.ndim() == 0 || b.ndim() == 0 || a.ndim() == b.ndim(),
                    "Arguments to binary operation '" + functor_name + "' must have the same rank (got left.ndim = " +
                        std::to_string(a.ndim()) + ", left.shape = " + shape_str(a.shape()) + ", and right.ndim = " +
                        std::to_string(b.ndim()) + ", right.shape = " + shape_str(b.shape()) + ").");
    }
    if (a.dtype() != b.dtype()) {
        DType t = type_promotion(a, b);
        a = astype(a, t);
        b = astype(b, t);
    }
    if (update_shape && a.shape() != b.shape()) {
        std::vector<int> cs = common_shape(a, b, functor_name);
        if (a.ndim() != 0) a = a.broadcast_to_shape(cs);
        if (b.ndim() != 0) b = b.broadcast_to_shape(cs);
    }
    return std::tuple<Array, Array>(a, b);
}

Array elementwise(Array a, Array b, const std::string& functor_name) {
    std::tie(a, b) = ensure_arguments_compatible(a, b, functor_name, true);
    const std::vector<int>& shape = a.ndim() == 0 ? b.shape() : a.shape();
    return Array(std::make_shared<Elementwise>(strip(functor_name), std::vector<Array>({a, b}), shape, a.dtype()));
}

Array unsafe_cast(Array a, DType type) {
    if (a.dtype() == type) return a;
    if (type == DTYPE_BF16) {
        // the float a bf16 store keeps; the node is typed bf16 so that evaluating it allocates 16-bit storage
        Array f = unsafe_cast(a, DTYPE_FLOAT);
        return Array(std::make_shared<Elementwise>("bf16_round", std::vector<Array>({f}), f.shape(), DTYPE_BF16));
    }
    if (ScalarValue* s = as<ScalarValue>(a)) {
        double v = s->value_;
        if (type == DTYPE_INT32) v = (double)(int)v;
        return Array(std::make_shared<ScalarValue>(v, type));
    }
    return Array(std::make_shared<Elementwise>("cast", std::vector<Array>({a}), a.shape(), type));
}
Array round(Array a) {
    if (a.dtype() == DTYPE_INT32) return a;
    a = computed_in_float(a);
    return Array(std::make_shared<Elementwise>("round", std::vector<Array>({a}), a.shape(), DTYPE_INT32));
}
Array ceil(Array a) {
    if (a.dtype() == DTYPE_INT32) return a;
    a = computed_in_float(a);
    return Array(std::make_shared<Elementwise>("ceiling", std::vector<Array>({a}), a.shape(), DTYPE_INT32));
}
Array astype(Array a, DType type) { return type == DTYPE_INT32 ? round(a) : unsafe_cast(a, type); }

Array identity(Array x) { return elementwise(x, "identity"); }
Array identity(int x) { return Array(x); }
Array identity(float x) { return Array(x); }
Array identity(double x) { return Array(x); }
#define DALI_UNARY(NAME, FUNCTOR) Array NAME(Array x) { return elementwise(x, FUNCTOR); }
DALI_UNARY(sqrt, "sqrt_f")
DALI_UNARY(square, "square")
DALI_UNARY(abs, "abs")
DALI_UNARY(sigmoid, "sigmoid")
DALI_UNARY(dsigmoid, "dsigmoid")
DALI_UNARY(tanh, "tanh")
DALI_UNARY(dtanh, "dtanh")
DALI_UNARY(relu, "relu")
DALI_UNARY(relu_backward, "relu_backward")
DALI_UNARY(eltinv, "inv")
DALI_UNARY(exp, "exp")
DALI_UNARY(log, "log")
DALI_UNARY(log_or_zero, "log_or_zero")
DALI_UNARY(sign, "sign")
DALI_UNARY(softplus, "softplus")
DALI_UNARY(softplus_backward, "softplus_backward")
DALI_UNARY(cube, "cube")
DALI_UNARY(rsqrt, "rsqrt")
DALI_UNARY(isnan, "isnotanumber")
DALI_UNARY(isinf, "isinfinity")
DALI_UNARY(inverse_tanh, "inverse_tanh")

#define DALI_BINARY(NAME, FUNCTOR) Array NAME(Array a, Array b) { return elementwise(a, b, FUNCTOR); }
DALI_BINARY(add, "add")
DALI_BINARY(subtract, "subtract")
DALI_BINARY(eltmul, "eltmul")
DALI_BINARY(eltdiv, "eltdiv")
DALI_BINARY(equals, "equals")
DALI_BINARY(pow, "power")
DALI_BINARY(steep_sigmoid, "steep_sigmoid")
DALI_BINARY(steep_sigmoid_backward, "steep_sigmoid_backward")
DALI_BINARY(clipped_relu, "clipped_relu")
DALI_BINARY(clipped_relu_backward, "clipped_relu_backward")
DALI_BINARY(prelu, "prelu")
DALI_BINARY(prelu_backward_weights, "prelu_backward_weights")
DALI_BINARY(prelu_backward_inputs, "prelu_backward_inputs")
DALI_BINARY(lessthanequal, "lessthanequal")
DALI_BINARY(greaterthanequal, "greaterthanequal")
DALI_BINARY(maximum, "max_scalar")
DALI_BINARY(minimum, "min_scalar")
DALI_BINARY(clip, "clip")
DALI_BINARY(binary_cross_entropy, "binary_cross_entropy")
DALI_BINARY(binary_cross_entropy_grad, "binary_cross_entropy_grad")

Array all_equals(Array l, Array r) { return op::prod(op::equals(l, r)); }
Array close(Array l, Array r, Array atol) { return op::lessthanequal(op::abs(op::subtract(l, r)), atol); }
Array all_close(Array l, Array r, Array atol) { return op::prod(op::close(l, r, atol)); }

Array add(const std::vector<Array>& arrays, bool) {
    DALI_ASSERT(!arrays.empty(), "add must have at least one Array to add but got 0.");
    Array out = arrays[0];
    for (size_t i = 1; i < arrays.size(); ++i) out = op::add(out, arrays[i]);
    return out;
}

Array fill(const Array& x, double value) {
    return Array(std::make_shared<Elementwise>("fill", std::vector<Array>({x, Array(value, x.dtype())}), x.shape(), x.dtype()));
}

// ---------------------------------------------------------------- reducers
static std::string reducer_short(const std::string& name) {
    const std::string pre = "reducers::";
    std::string n = name.compare(0, pre.size(), pre) == 0 ? name.substr(pre.size()) : name;
    if (n == "maximum") return "max";
    if (n == "minimum") return "min";
    if (n == "product") return "prod";
    return n;
}

Array all_reduce(const Array& a_in, const std::string& reducer_name) {
    DALI_ASSERT(!a_in.is_stateless(), "reduction of a stateless Array");
    const Array a = computed_in_float(a_in);
    if (a.ndim() == 0) return a;
    return Array(std::make_shared<Reduce>(reducer_short(reducer_name), a, a.ndim(), false, a.dtype()));
}

Array axis_reduce(const Array& a_in, const std::string& reducer_name, const std::vector<int>& axes, bool keepdims) {
    DALI_ASSERT(!a_in.is_stateless(), "reduction of a stateless Array");
    const Array a = computed_in_float(a_in);
    if (axes.empty()) return a;
    const int ndim = a.ndim();
    if (ndim == 0) return a;
    std::vector<int> norm(axes);
    std::vector<bool> reduced(ndim, false);
    for (int& axis : norm) {
        if (axis < 0) axis += ndim;
        DALI_ASSERT(axis >= 0 && axis < ndim,
                    "Reduction axis must strictly positive and less than the number of dimensions of the input (got axis=" +
                        std::to_string(axes[0]) + ", ndim=" + std::to_string(ndim) + ", input.shape = " + shape_str(a.shape()) + ").");
    }
    std::sort(norm.begin(), norm.end());
    for (int axis : norm) {
        DALI_ASSERT(!reduced[axis], "axis_reduce received duplicate axes to operate on (axis=" + std::to_string(axis) + ").");
        reduced[axis] = true;
    }
    Array res;
    if ((int)norm.size() == ndim) {
        res = all_reduce(a, reducer_name);
    } else {
        // kept axes first, reduced axes last (a view -- no data moves), then fold the tail
        std::vector<int> order;
        for (int d = 0; d < ndim; ++d) if (!reduced[d]) order.push_back(d);
        for (int d = 0; d < ndim; ++d) if (reduced[d]) order.push_back(d);
        bool is_identity = true;
        for (int d = 0; d < ndim; ++d) is_identity = is_identity && order[d] == d;
        Array moved = is_identity ? a : a.transpose(order);
        res = Array(std::make_shared<Reduce>(reducer_short(reducer_name), moved, (int)norm.size(), false, a.dtype()));
    }
    if (keepdims) for (int axis : norm) res = res.expand_dims(axis);
    return res;
}

Array argument_all_reduce(const Array& a_in, const std::string& reducer_name) {
    DALI_ASSERT(!a_in.is_stateless(), "reduction of a stateless Array");
    const Array a = computed_in_float(a_in);
    if (a.ndim() == 0) return Array(0);
    // int32, where the reference mistypes the result as the input's dtype
    // (dali/array/op/reducer_operation.cpp:681-684)
    return Array(std::make_shared<Reduce>(reducer_short(reducer_name), a, a.ndim(), true, DTYPE_INT32));
}

Array argument_axis_reduce(const Array& a_in, const std::string& reducer_name, const int& axis) {
    const Array a = computed_in_float(a_in);
    const int ndim = a.ndim();
    if (ndim == 0) return Array(0);
    int norm = axis < 0 ? axis + ndim : axis;
    DALI_ASSERT(norm >= 0 && norm < ndim,
                "Reduction axis must strictly positive and less than the number of dimensions of the input (got axis=" +
                    std::to_string(norm) + ", ndim=" + std::to_string(ndim) + ").");
    if (ndim == 1) return argument_all_reduce(a, reducer_name);
    Array moved = a;
    if (norm != ndim - 1) {
        // kept axes stay in order, the searched axis goes last
        std::vector<int> order;
        for (int d = 0; d < ndim; ++d) if (d != norm) order.push_back(d);
        order.push_back(norm);
        moved = a.transpose(order);
    }
    return Array(std::make_shared<Reduce>(reducer_short(reducer_name), moved, 1, true, DTYPE_INT32));
}

Array sum(const Array& x) { return all_reduce(x, "sum"); }
Array sum(const Array& x, const std::vector<int>& axes, bool k) { return axis_reduce(x, "sum", axes, k); }
Array prod(const Array& x) { return all_reduce(x, "prod"); }
Array prod(const Array& x, const std::vector<int>& axes, bool k) { return axis_reduce(x, "prod", axes, k); }
Array max(const Array& x) { return all_reduce(x, "max"); }
Array max(const Array& x, const std::vector<int>& axes, bool k) { return axis_reduce(x, "max", axes, k); }
Array min(const Array& x) { return all_reduce(x, "min"); }
Array min(const Array& x, const std::vector<int>& axes, bool k) { return axis_reduce(x, "min", axes, k); }
Array mean(const Array& x) {
    Array s = all_reduce(x, "sum");
    if (s.dtype() == DTYPE_INT32) s = astype(s, DTYPE_DOUBLE);
    return op::eltdiv(s, Array((int)lazy::global_numel(x)));     // (of the logical array when x is one rank's shard)
}
Array mean(const Array& x, const std::vector<int>& axes, bool k) {
    Array s = axis_reduce(x, "sum", axes, k);
    if (s.dtype() == DTYPE_INT32) s = astype(s, DTYPE_DOUBLE);
    return op::eltdiv(s, Array((int)(lazy::global_numel(x) / std::max<int64_t>(1, lazy::global_numel(s)))));
}
Array L2_norm(const Array& x) {
    Array s = all_reduce(op::square(x), "sum");
    if (s.dtype() == DTYPE_INT32) s = astype(s, DTYPE_DOUBLE);
    return op::sqrt(s);
}
Array L2_norm(const Array& x, const std::vector<int>& axes, bool k) {
    Array s = axis_reduce(op::square(x), "sum", axes, k);
    if (s.dtype() == DTYPE_INT32) s = astype(s, DTYPE_DOUBLE);
    return op::sqrt(s);
}
Array argmax(const Array& x) { return argument_all_reduce(x, "max"); }
Array argmax(const Array& x, const int& axis) { return argument_axis_reduce(x, "max", axis); }
Array argmin(const Array& x) { return argument_all_reduce(x, "min"); }
Array argmin(const Array& x, const int& axis) { return argument_axis_reduce(x, "min", axis); }
Array any_isnan(const Array& a) { return op::max(op::isnan(a)); }
Array any_isinf(const Array& a) { return op::max(op::isinf(a)); }
Array any_isnan(const Array& a, const std::vector<int>& axes, bool k) { return op::max(op::isnan(a), axes, k); }
Array any_isinf(const Array& a, const std::vector<int>& axes, bool k) { return op::max(op::isinf(a), axes, k); }

// ---------------------------------------------------------------- index ops
Array gather(const Array& source, const Array& indices) {
    DALI_ASSERT(source.ndim() > 0, "gather must be called on source with ndim >= 1 (got ndim=" + std::to_string(source.ndim()) + ").");
    DALI_ASSERT(indices.dtype() == DTYPE_INT32, "indices must be integers (got dtype=" + dtype_to_name(indices.dtype()) + ").");
    return Array(std::make_shared<Gather>(source, indices));
}
Array gather_from_rows(const Array& source, const Array& indices) {
    DALI_ASSERT(source.ndim() > 1, "gather_from_rows must be called on source with ndim >= 2 (got ndim=" + std::to_string(source.ndim()) + ").");
    DALI_ASSERT(indices.dtype() == DTYPE_INT32, "indices must be integers (got dtype=" + dtype_to_name(indices.dtype()) + ").");
    DALI_ASSERT(indices.ndim() <= 1, "indices must have rank 1 or lower [Note: support for higher ranks coming soon] (got indices.ndim=" + std::to_string(indices.ndim()) + ").");
    Array idx = indices;
    if (idx.ndim() == 0) idx = idx.expand_dims(0).broadcast_to_shape({source.shape()[0]});
    DALI_ASSERT(idx.shape()[0] <= source.shape()[0], "indices cannot have a larger first dimension than source");
    Array src = source;
    if (idx.shape()[0] < source.shape()[0]) src = source.pluck_axis(0, Slice(0, idx.shape()[0]));
    return Array(std::make_shared<GatherFromRows>(src, idx));
}

// ---------------------------------------------------------------- compositions
Array softmax(const Array& logits, int axis) {
    Array exped = op::exp(logits - op::max(logits, {axis}, true));
    return exped / op::sum(exped, {axis}, true);
}
Array softmax_temperature(const Array& logits, const Array&, int axis) {
    // the reference ignores its temperature argument (dali/array/op/softmax.cpp:10-13)
    return softmax(logits, axis);
}

// ---------------------------------------------------------------- dot
Array matmul(Array a, Array b) {
    DALI_ASSERT(a.ndim() == 2 && b.ndim() == 2, "matmul inputs must be matrices (got left.ndim = " + std::to_string(a.ndim()) + ", right.ndim = " + std::to_string(b.ndim()) + ").");
    DALI_ASSERT(a.shape()[1] == b.shape()[0] || a.shape()[1] == 1 || b.shape()[0] == 1,
                "shapes " + shape_str(a.shape()) + " and " + shape_str(b.shape()) + " not aligned: " +
                    std::to_string(a.shape()[1]) + " (dim 1) != " + std::to_string(b.shape()[0]) + " (dim 0)");
    if (a.shape()[1] != b.shape()[0]) {
        // a size-1 inner dim broadcasts (dali/array/op/dot.cpp:47-61)
        if (a.shape()[1] == 1) a = a.broadcast_to_shape({a.shape()[0], b.shape()[0]});
        else b = b.broadcast_to_shape({a.shape()[1], b.shape()[1]});
    }
    if (a.dtype() != b.dtype()) {
        DType t = type_promotion(a, b);
        a = astype(a, t);
        b = astype(b, t);
    }
    return Array(std::make_shared<MatMul>(a, b));
}
Array matrix_vector_dot(const Array& a, const Array& b) {
    if (a.ndim() == 1 && b.ndim() == 2) return matmul(a.expand_dims(0), b).squeeze(0);
    DALI_ASSERT(a.ndim() == 2 && b.ndim() == 1, "matrix_vector_dot takes a matrix and a vector");
    return matmul(a, b.expand_dims(1)).squeeze(1);
}
Array inner(const Array& a, const Array& b) {
    DALI_ASSERT(a.ndim() == 1 && b.ndim() == 1, "inner takes two vectors");
    return matmul(a.expand_dims(0), b.expand_dims(1)).squeeze(1).squeeze(0);
}
Array dot(const Array& a, const Array& b) {
    int an = a.ndim(), bn = b.ndim();
    if (an == 0 || bn == 0) return a * b;
    if (an == 1 && bn == 1) return inner(a, b);
    if (an == 2 && bn == 2) return matmul(a, b);
    if ((an == 1 && bn == 2) || (an == 2 && bn == 1)) return matrix_vector_dot(a, b);
    throw std::runtime_error("dot of arrays with rank above 2 (tensordot) is not part of this back end");
}

// ---------------------------------------------------------------- arange, eye, one_hot, outer, scan
Array arange(int start, int stop, int step) {
    DALI_ASSERT(step != 0, "arange's step cannot be zero.");
    // size = (int)ceil((stop - start) / step) in the operands' type (dali/array/op/arange.cpp:63):
    // with three ints the division truncates, so arange(0, 10, 3) has 3 elements
    const int n = (stop - start) / step;
    DALI_ASSERT(n > 0, "arange's size must be strictly positive (got start = " + std::to_string(start) + ", stop = " +
                           std::to_string(stop) + ", step = " + std::to_string(step) + ").");
    return Array(std::make_shared<Iota>(std::vector<int>({n}), (int64_t)start, std::vector<int64_t>({(int64_t)step})));
}
Array arange(int start, int stop) { return arange(start, stop, 1); }
Array arange(int stop) { return arange(0, stop, 1); }
Array arange(const Array& start, const Array& stop, const Array& step) {
    DALI_ASSERT(start.ndim() == 0, "arange's start argument must be a scalar but got start.shape = " + shape_str(start.shape()) + ".");
    DALI_ASSERT(stop.ndim() == 0, "arange's stop argument must be a scalar but got stop.shape = " + shape_str(stop.shape()) + ".");
    DALI_ASSERT(step.ndim() == 0, "arange's step argument must be a scalar but got step.shape = " + shape_str(step.shape()) + ".");
    const double a = (double)start, b = (double)stop, st = (double)step;
    const bool ints = start.dtype() == DTYPE_INT32 && stop.dtype() == DTYPE_INT32 && step.dtype() == DTYPE_INT32;
    DALI_ASSERT(st != 0, "arange's step cannot be zero.");
    // the quotient is formed in the operands' common type: integer operands truncate (arange.cpp:63)
    const int size = ints ? ((int)b - (int)a) / (int)st : (int)std::ceil((b - a) / st);
    DALI_ASSERT(size > 0, "arange's size must be strictly positive (got start = " + std::to_string(a) + ", stop = " +
                              std::to_string(b) + ", step = " + std::to_string(st) + ").");
    if (ints)
        return Array(std::make_shared<Iota>(std::vector<int>({size}), (int64_t)a, std::vector<int64_t>({(int64_t)st})));
    // start + index * step in start's type (dali/array/op/arange.cpp:41)
    Array idx(std::make_shared<Iota>(std::vector<int>({size}), 0, std::vector<int64_t>({1})));
    return unsafe_cast(start + unsafe_cast(idx, start.dtype()) * unsafe_cast(step, start.dtype()), start.dtype());
}

Array eye(int size) { return eye(size, size); }
Array eye(int rows, int cols) {
    DALI_ASSERT(rows > 0 && cols > 0, "eye's rows and cols must > 0 (got rows = " + std::to_string(rows) + ", cols = " + std::to_string(cols) + ").");
    return diag(Array(1.0f), rows, cols);
}
Array diag(const Array& d) {
    DALI_ASSERT(d.ndim() == 1, "diag with no size needs a vector");
    return diag(d, d.shape()[0], d.shape()[0]);
}
Array diag(const Array& d, int rows) { return diag(d, rows, rows); }
Array diag(const Array& d, int rows, int cols) {
    DALI_ASSERT(rows > 0 && cols > 0, "diag's rows and cols must > 0 (got rows = " + std::to_string(rows) + ", cols = " + std::to_string(cols) + ").");
    DALI_ASSERT(d.ndim() <= 1, "diag's argument must be a scalar or a vector (got array.shape = " + shape_str(d.shape()) + ").");
    const int m = std::min(rows, cols);
    if (d.ndim() == 1)
        DALI_ASSERT(d.shape()[0] >= m, "diag's argument is smaller than the maximal diagonal item (array.shape = " +
                                           shape_str(d.shape()) + ", rows = " + std::to_string(rows) + ", cols = " + std::to_string(cols) + ").");
    const std::vector<int> shape({rows, cols});
    Array i(std::make_shared<Iota>(shape, 0, std::vector<int64_t>({1, 0})));
    Array j(std::make_shared<Iota>(shape, 0, std::vector<int64_t>({0, 1})));
    Array on_diag = unsafe_cast(elementwise(i, j, "equals"), d.dtype());
    Array values = d;
    if (d.ndim() == 1) {
        // only entries below min(rows, cols) are ever selected: view whichever side is long enough
        if (d.shape()[0] >= cols) values = d.pluck_axis(0, Slice(0, cols)).expand_dims(0).broadcast_to_shape(shape);
        else values = d.pluck_axis(0, Slice(0, rows)).expand_dims(1).broadcast_to_shape(shape);
    }
    return elementwise(on_diag, values, "where_nonzero");
}

Array one_hot(const Array& indices, int depth, const Array& on_value, const Array& off_value) {
    DALI_ASSERT(indices.dtype() == DTYPE_INT32, "indices must be integers (got " + dtype_to_name(indices.dtype()) + ").");
    DALI_ASSERT(on_value.ndim() == 0, "on_value must be a scalar (got on_value.ndim=" + std::to_string(on_value.ndim()) + ").");
    DALI_ASSERT(off_value.ndim() == 0, "off_value must be a scalar (got off_value.ndim=" + std::to_string(off_value.ndim()) + ").");
    DALI_ASSERT(depth > 0, "depth must be strictly positive (got depth=" + std::to_string(depth) + ").");
    std::vector<int> shape = indices.shape();
    shape.push_back(depth);
    std::vector<int64_t> st(shape.size(), 0);
    st.back() = 1;
    Array position(std::make_shared<Iota>(shape, 0, st));
    Array idx = indices.expand_dims(indices.ndim()).broadcast_to_shape(shape);
    const DType t = on_value.dtype();
    // on * is_on + (1 - is_on) * off, as the reference's kernel writes it (one_hot.cpp:45-46)
    Array is_on = unsafe_cast(elementwise(idx, position, "equals"), t);
    Array off = unsafe_cast(off_value, t);
    return on_value * is_on + (unsafe_cast(Array(1.0), t) - is_on) * off;
}

Array outer(const Array& a_, const Array& b_) {
    Array a = a_.ravel(), b = b_.ravel();
    std::tie(a, b) = ensure_arguments_compatible(a, b, "outer", /*update_shape=*/false);
    const std::vector<int> shape({a.shape()[0], b.shape()[0]});
    return elementwise(a.expand_dims(1).broadcast_to_shape(shape), b.expand_dims(0).broadcast_to_shape(shape), "eltmul");
}

Array axis_scan(const Array& a, const std::string& reducer_name, bool inclusive) {
    std::string r = reducer_name;
    if (r.compare(0, 10, "reducers::") == 0) r = r.substr(10);
    if (r == "maximum") r = "max";
    if (r == "minimum") r = "min";
    if (r == "product") r = "prod";
    DALI_ASSERT(r == "sum" || r == "prod" || r == "max" || r == "min", "axis_scan: unknown reducer " + reducer_name);
    Array x = computed_in_float(a.ndim() == 0 ? a.expand_dims(0) : a);
    return Array(std::make_shared<Scan>(x, r, inclusive));
}
Array cumsum(const Array& a, bool inclusive) { return axis_scan(a, "reducers::sum", inclusive); }
Array cumprod(const Array& a, bool inclusive) { return axis_scan(a, "reducers::product", inclusive); }

// ---------------------------------------------------------------- random numbers
namespace {
// value of element i = functor(i, seed): an Elementwise over (row-major index, seed drawn now)
Array random_field(const char* functor, const std::vector<int>& shape, DType dtype) {
    for (int d : shape) DALI_ASSERT(d >= 0, "random: negative dimension");
    std::vector<int64_t> st(shape.size(), 0);
    int64_t acc = 1;
    for (int d = (int)shape.size() - 1; d >= 0; --d) { st[d] = acc; acc *= shape[d]; }
    DALI_ASSERT(acc <= 2147483647LL, "random: more than 2^31 - 1 elements in one array");
    Array index(std::make_shared<Iota>(shape, 0, st));
    Array seed(std::make_shared<ScalarValue>((double)utils::randint(0, 2147483646), DTYPE_INT32));
    return Array(std::make_shared<Elementwise>(functor, std::vector<Array>({index, seed}), shape, dtype));
}
#define DALI_ASSERT_SCALAR(NAME, ARG, ARRAY) \
    DALI_ASSERT(ARRAY.ndim() == 0, std::string(NAME) + "'s " + ARG + " argument must be a scalar but got " + ARG + ".shape = " + shape_str(ARRAY.shape()) + ".")
}  // namespace

Array uniform(Array low, Array high, const std::vector<int>& shape) {
    DALI_ASSERT_SCALAR("uniform", "low", low);
    DALI_ASSERT_SCALAR("uniform", "high", high);
    std::tie(low, high) = ensure_arguments_compatible(low, high, "uniform", false);
    const DType t = low.dtype();
    if (t == DTYPE_INT32) {
        // inclusive range, as std::uniform_int_distribution (random.cu.cpp:67-74): low + floor(u * (high - low + 1))
        Array u = random_field("rng_uniform", shape, DTYPE_DOUBLE);
        Array span = unsafe_cast(high - low, DTYPE_DOUBLE) + Array(1.0);
        return low + unsafe_cast(u * span, DTYPE_INT32);
    }
    return low + (high - low) * random_field("rng_uniform", shape, t);
}
Array normal(Array loc, Array scale, const std::vector<int>& shape) {
    DALI_ASSERT_SCALAR("normal", "loc", loc);
    DALI_ASSERT_SCALAR("normal", "scale", scale);
    if (loc.dtype() == DTYPE_INT32) loc = unsafe_cast(loc, DTYPE_DOUBLE);
    if (scale.dtype() == DTYPE_INT32) scale = unsafe_cast(scale, DTYPE_DOUBLE);
    std::tie(loc, scale) = ensure_arguments_compatible(loc, scale, "normal", false);
    return loc + scale * random_field("rng_normal", shape, loc.dtype());
}
Array bernoulli(Array prob, const std::vector<int>& shape) {
    DALI_ASSERT_SCALAR("bernoulli", "prob", prob);
    if (prob.dtype() == DTYPE_INT32) prob = unsafe_cast(prob, DTYPE_DOUBLE);
    // uniform(0, 1) <= prob (random.cu.cpp:316-320)
    return lessthanequal(random_field("rng_uniform", shape, prob.dtype()), prob);
}
Array bernoulli_normalized(Array prob, const std::vector<int>& shape) {
    return bernoulli(prob, shape) * eltinv(prob.dtype() == DTYPE_INT32 ? unsafe_cast(prob, DTYPE_DOUBLE) : prob);
}

Array control_dependency(Array condition, Array result) {
    if (!condition.is_stateless() && !condition.is_buffer()) condition.eval(false);
    return result;
}

// ---------------------------------------------------------------- concatenate
// The pieces are written into consecutive slices of one new array (reference: dali/array/op/concatenate.cpp:10-73,
// a ControlFlow node over one assignment per piece).  Here the assignments are evaluated together when the call is
// made; dims of size 1 outside the axis broadcast to the common shape as in the reference.
Array concatenate(const std::vector<Array>& arrays, int axis) {
    DALI_ASSERT(!arrays.empty(), "concatenate must receive at least one array.");
    if (arrays.size() == 1) return arrays[0];
    const int ndim = arrays[0].ndim();
    DALI_ASSERT(ndim > 0, "concatenate requires arrays with ndim > 0 (got " + arrays[0].expression_name() + ").");
    if (axis < 0) axis += ndim;
    DALI_ASSERT(axis >= 0 && axis < ndim, "concatenation axis must be >= 0 and < arrays[0].ndim = " + std::to_string(ndim) +
                                              ", but got axis = " + std::to_string(axis) + ".");
    std::vector<int> common = arrays[0].shape();
    int total = 0;
    for (const Array& a : arrays) {
        DALI_ASSERT(a.ndim() == ndim, "all the input arrays must have the same dimensionality (expected ndim = " +
                                          std::to_string(ndim) + ", got " + std::to_string(a.ndim()) + ").");
        for (int d = 0; d < ndim; ++d) {
            if (d == axis) continue;
            if (common[d] == 1) common[d] = a.shape()[d];
            DALI_ASSERT(common[d] == a.shape()[d] || a.shape()[d] == 1,
                        "all the input array dimensions must match exactly outside of the concatenation axis, but got " +
                            a.expression_name() + ".");
        }
        total += a.shape()[axis];
    }
    std::vector<int> out_shape = common;
    out_shape[axis] = total;
    Array result(out_shape, arrays[0].dtype(), arrays[0].preferred_device());
    std::vector<Array> assignments;
    int so_far = 0;
    for (Array a : arrays) {
        common[axis] = a.shape()[axis];
        if (a.shape() != common) a = a.broadcast_to_shape(common);
        assignments.push_back(op::assign(result.pluck_axis(axis, Slice(so_far, so_far + common[axis])), OPERATOR_T_EQL, a));
        so_far += common[axis];
    }
    Array::eval_together(assignments, false);
    return result;
}
Array hstack(const std::vector<Array>& arrays) { return concatenate(arrays, -1); }
Array vstack(const std::vector<Array>& arrays) { return concatenate(arrays, 0); }

// ---------------------------------------------------------------- assignment
Array assign(const Array& left, OPERATOR_T op, const Array& right) {
    if (op == OPERATOR_T_LSE) return autoreduce_assign(left, right);
    return Array(std::make_shared<Assignment>(left, op, right));
}
Array autoreduce_assign(const Array& left, const Array& right) {
    DALI_ASSERT(left.ndim() == right.ndim(),
                "destination for autoreduce_assign must have the same dimensionality as the input (destination.ndim = " +
                    std::to_string(left.ndim()) + " vs input.ndim = " + std::to_string(right.ndim()));
    std::vector<int> axes;
    for (int d = 0; d < right.ndim(); ++d) {
        if (left.shape()[d] != right.shape()[d]) {
            DALI_ASSERT(left.shape()[d] == 1, "Could not autoreduce_assign: destination must have all dimensions equal input dimensions or equal 1, but destination.shape[" + std::to_string(d) + "] = " + std::to_string(left.shape()[d]) + " vs input.shape[" + std::to_string(d) + "] = " + std::to_string(right.shape()[d]));
            axes.push_back(d);
        }
    }
    Array r = axes.empty() ? right : op::sum(right, axes, true);
    return Array(std::make_shared<Assignment>(Array(left.expression()), OPERATOR_T_ADD, r));
}
Array to_assignment(const Array& node) {
    return Array(std::make_shared<Assignment>(Array(node.shape(), node.dtype(), node.preferred_device()), OPERATOR_T_EQL,
                                              Array(node.expression())));
}

}  // namespace op
