// The plug-in seam between the expression graph and whatever runs it (reference:
// dali/array/expression/computation.h:7-38, computation.cpp:13-28,47-165).
//
// Array::eval makes the value an assignment (canonical, optimization.h), turns it into Computations with
// convert_to_ops and calls run_and_cleanup on each.  Which Computation runs an assignment is looked up the way the
// reference does it: factories registered for the typeid name of the right-hand side's node class first, then the
// (name, predicate) ones, the first factory that returns a non-null Computation wins; what nobody claims goes to the
// built-in implementations -- the fused-kernel lowering for everything a generated kernel can express, the GEMM entry
// points for a product.  A factory declines by returning nullptr.  The node classes a factory can match on
// (Elementwise, Reduce, MatMul, View, Gather, ...) are declared in dali/array/expression/expression.h.
#ifndef DALI_ARRAY_EXPRESSION_COMPUTATION_H
#define DALI_ARRAY_EXPRESSION_COMPUTATION_H

#include <functional>
#include <memory>
#include <string>
#include <typeinfo>
#include <vector>

#include "dali/array/array.h"

struct Computation {
    Array left_;                // destination: a buffer view, or a gather of one (scatter)
    OPERATOR_T operator_t_;
    Array right_;               // the value
    Array assignment_;          // the handle that stands for "left (op)= right"; becomes the destination afterwards

    Computation(Array left, OPERATOR_T operator_t, Array right, Array assignment);
    virtual ~Computation() {}
    virtual void run() = 0;
    // run() inside a trace scope named after the value, then the assignment is replaced by its destination: the
    // result is remembered in the graph and never computed again
    void run_and_cleanup();
    // destination / i-th argument of the value as device (or host) pointers at the element the view starts at,
    // made fresh on `device` first (computation.cpp:122-132)
    void* left_data(memory::Device device);
    const void* argument_data(memory::Device device, int idx) const;
};

typedef std::function<std::shared_ptr<Computation>(Array, OPERATOR_T, Array, Array)> to_computation_t;
typedef std::function<bool(const Array&)> implementation_test_t;

int register_implementation(const char* opname, to_computation_t impl);
int register_implementation(const std::string& opname, implementation_test_t test, to_computation_t impl);

// execution order; `root` has been through canonical()
std::vector<std::shared_ptr<Computation>> convert_to_ops(Array root);

template <typename ExpressionT, typename Comp>
int register_implementation_default() {
    return register_implementation(typeid(ExpressionT).name(),
                                   [](Array dest, OPERATOR_T operator_t, Array x, Array assignment) -> std::shared_ptr<Computation> {
                                       return std::make_shared<Comp>(dest, operator_t, x, assignment);
                                   });
}

#endif
