// Test infrastructure only.  Array operators that the reference's autodiff layer can call but that are not on the
// lazy-expression path of the B200 back end: declared here so that the reference's translation units compile,
// defined in ../../../../shims.cpp, where every one of them throws std::runtime_error when reached.
#ifndef DALI_B200_ORACLE_OFF_PATH_OPS_H
#define DALI_B200_ORACLE_OFF_PATH_OPS_H

#include "dali/array/array.h"

namespace op {
// sorting (reference: dali/array/op/top_k.h)
Array top_k(const Array& array, int k, bool sorted = true);
Array bottom_k(const Array& array, int k, bool sorted = true);
Array argsort(const Array& array);
Array argsort(const Array& array, int axis);
// reference: dali/array/op/circular_convolution.h
Array circular_convolution(Array x, Array weights);
}  // namespace op

#endif
