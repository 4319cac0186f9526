// Test infrastructure only -- not part of the shipped library.
//
// The reference's autodiff layer (dali/tensor) also calls a few Array operators
// that are not on the lazy-expression path and that the B200 back end does not
// provide: sorting (op/top_k.h) and circular convolution.  Their declarations
// are in include/ beside this file; the definitions here exist so that the
// reference's translation units link, and throw when reached.
#include <stdexcept>

#include <string>

#include "dali/array/op/off_path_ops.h"

namespace {
[[noreturn]] void off_path(const char* name) {
    throw std::runtime_error(std::string(name) + " is not part of the lazy-expression path of the B200 back end");
}
}  // namespace

namespace op {
Array top_k(const Array&, int, bool) { off_path("op::top_k"); }
Array bottom_k(const Array&, int, bool) { off_path("op::bottom_k"); }
Array argsort(const Array&) { off_path("op::argsort"); }
Array argsort(const Array&, int) { off_path("op::argsort"); }
Array circular_convolution(Array, Array) { off_path("op::circular_convolution"); }
}  // namespace op
