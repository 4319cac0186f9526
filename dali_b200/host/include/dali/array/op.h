// op:: free functions of the lazy front end (reference: dali/array/op.h umbrella,
// op/unary.h:7-31, op/binary.h:6-32, op/reducers.h:8-47, op/elementwise_operation.h,
// op/gather.h, op/gather_from_rows.h, op/softmax.h, op/dot.h, op/arange.h).
#ifndef DALI_ARRAY_OP_H
#define DALI_ARRAY_OP_H

#include <string>
#include <tuple>
#include <vector>

#include "dali/array/array.h"

namespace op {
// ---- elementwise (functor names as in dali/array/functor.h)
Array elementwise(Array a, const std::string& functor_name);
Array elementwise(Array a, Array b, const std::string& functor_name);
Array astype(Array x, DType dtype);          // rounds when converting to int32
Array unsafe_cast(Array x, DType dtype);     // static_cast
Array round(Array x);
Array ceil(Array x);
std::tuple<Array, Array> ensure_arguments_compatible(Array a, Array b, const std::string& functor_name, bool update_shape);

Array identity(Array x);
Array identity(int x);
Array identity(float x);
Array identity(double x);
Array sqrt(Array x);
Array square(Array x);
Array abs(Array x);
Array sigmoid(Array x);
Array dsigmoid(Array x);
Array tanh(Array x);
Array dtanh(Array x);
Array relu(Array x);
Array relu_backward(Array x);
Array eltinv(Array x);
Array exp(Array x);
Array log(Array x);
Array log_or_zero(Array x);
Array sign(Array x);
Array softplus(Array x);
Array softplus_backward(Array x);
Array cube(Array x);
Array rsqrt(Array x);
Array isnan(Array x);
Array isinf(Array x);
Array inverse_tanh(Array x);

Array all_equals(Array left, Array right);
Array all_close(Array left, Array right, Array atolerance);
Array close(Array left, Array right, Array atolerance);
Array add(Array left, Array right);
Array add(const std::vector<Array>& arrays, bool single_op = false);
Array subtract(Array left, Array right);
Array eltmul(Array left, Array right);
Array eltdiv(Array left, Array right);
Array equals(Array left, Array right);
Array pow(Array left, Array right);
Array steep_sigmoid(Array x, Array aggressiveness);
Array steep_sigmoid_backward(Array x, Array aggressiveness);
Array clipped_relu(Array x, Array clipval);
Array clipped_relu_backward(Array x, Array clipval);
Array prelu(Array x, Array weights);
Array prelu_backward_weights(Array a, Array grad);
Array prelu_backward_inputs(Array a, Array weights);
Array lessthanequal(Array a, Array b);
Array greaterthanequal(Array a, Array b);
Array maximum(Array a, Array b);
Array minimum(Array a, Array b);
Array clip(Array a, Array b);
Array binary_cross_entropy(Array a, Array b);
Array binary_cross_entropy_grad(Array a, Array b);

// ---- reducers
Array sum(const Array& x);
Array sum(const Array& x, const std::vector<int>& axes, bool keepdims = false);
Array prod(const Array& x);
Array prod(const Array& x, const std::vector<int>& axes, bool keepdims = false);
Array max(const Array& x);
Array max(const Array& x, const std::vector<int>& axes, bool keepdims = false);
Array min(const Array& x);
Array min(const Array& x, const std::vector<int>& axes, bool keepdims = false);
Array mean(const Array& x);
Array mean(const Array& x, const std::vector<int>& axes, bool keepdims = false);
Array L2_norm(const Array& x);
Array L2_norm(const Array& x, const std::vector<int>& axes, bool keepdims = false);
Array argmax(const Array& x);
Array argmax(const Array& x, const int& axis);
Array argmin(const Array& x);
Array argmin(const Array& x, const int& axis);
Array any_isnan(const Array& array);
Array any_isinf(const Array& array);
Array any_isnan(const Array& array, const std::vector<int>& axes, bool keepdims = false);
Array any_isinf(const Array& array, const std::vector<int>& axes, bool keepdims = false);
Array all_reduce(const Array& a, const std::string& reducer_name);
Array axis_reduce(const Array& a, const std::string& reducer_name, const std::vector<int>& axes, bool keepdims = false);
Array argument_all_reduce(const Array& a, const std::string& reducer_name);
Array argument_axis_reduce(const Array& a, const std::string& reducer_name, const int& axis);

// ---- index ops
Array gather(const Array& source, const Array& indices);
Array gather_from_rows(const Array& source, const Array& indices);

// ---- compositions
Array softmax(const Array& logits, int axis = -1);
Array softmax_temperature(const Array& logits, const Array& temperature, int axis = -1);

// ---- dot
Array matmul(Array a, Array b);
Array matrix_vector_dot(const Array& a, const Array& b);
Array inner(const Array& a, const Array& b);
Array dot(const Array& a, const Array& b);

// ---- construction helpers the reference's tests lean on
// lazy: an affine index expression, no memory until something evaluates it (op/arange.h)
Array arange(int start, int stop, int step);
Array arange(int start, int stop);
Array arange(int stop);
Array arange(const Array& start, const Array& stop, const Array& step);   // scalars; dtype of `start`
// op/eye.h: value[i, j] = i == j ? diag[j] : 0 (diag a scalar or a vector)
Array eye(int size);
Array eye(int rows, int cols);
Array diag(const Array& diag);
Array diag(const Array& diag, int rows);
Array diag(const Array& diag, int rows, int cols);
// op/one_hot.h: out[..., d] = indices[...] == d ? on_value : off_value, dtype of on_value
Array one_hot(const Array& indices, int depth, const Array& on_value, const Array& off_value);
// op/outer.h: out[i, j] = a.ravel()[i] * b.ravel()[j]
Array outer(const Array& a, const Array& b);
// op/concatenate.h: the arrays one after another along `axis` (negative counts from the back)
Array concatenate(const std::vector<Array>& arrays, int axis = 0);
Array hstack(const std::vector<Array>& arrays);      // axis -1
Array vstack(const std::vector<Array>& arrays);      // axis 0
// op/scan.h: running reduction over the last dim; exclusive results are one element longer
Array axis_scan(const Array& a, const std::string& reducer_name, bool inclusive);
Array cumsum(const Array& a, bool inclusive = true);
Array cumprod(const Array& a, bool inclusive = true);
Array fill(const Array& x, double value);      // same-shaped array holding `value`

// ---- random numbers (op/random.h:7-10).  low / high / loc / scale / prob are scalars.  Lazy: the value of
// element i is a pure function of (i, the seed drawn when the node was built), generated inside the
// kernel that consumes it.  uniform: [low, high) for float / double, [low, high] for int32.
Array uniform(Array low, Array high, const std::vector<int>& shape);
Array normal(Array loc, Array scale, const std::vector<int>& shape);
Array bernoulli(Array prob, const std::vector<int>& shape);
Array bernoulli_normalized(Array prob, const std::vector<int>& shape);

// expression/control_flow.h:33: `result`, evaluated no earlier than `condition`.  The reference threads a
// ControlFlow node through views of pending assignments; here a pending assignment is run when something first looks
// through it, so the dependency is discharged at once: `condition` is evaluated now and `result` returned as it is.
Array control_dependency(Array condition, Array result);

// ---- assignment
Array assign(const Array& left, OPERATOR_T operator_t, const Array& right);
Array autoreduce_assign(const Array& left, const Array& right);
Array to_assignment(const Array& node);
}  // namespace op

#endif
