// Test infrastructure only: force-included when building the reference's CPU
// path with a current g++.  Standard headers that libstdc++ no longer pulls in
// transitively, plus the ASSERT_SCALAR macro that dali/array/op/random.cu.cpp
// defines only inside its CUDA branch (:234-237) but uses unconditionally
// (:308-327).
#include <string>
#include <cstdint>
#include <cstring>
#include <functional>
#include "dali/utils/print_utils.h"
#ifndef ASSERT_SCALAR
#define ASSERT_SCALAR(name, array_name, array) \
    ASSERT2((array).ndim() == 0, utils::make_message(name, "'s ", array_name, \
        " argument must be a scalar but got ", array_name, ".shape = ", (array).shape(), "."));
#endif
