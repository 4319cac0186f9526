// Test infrastructure only -- not part of the shipped library.
// Headers of the reference-side binding (jit_b200_binding.inc, gemm_b200_binding.inc); oracle/build_ref.sh puts this
// include on the first line of the patched copies of dali/array/jit/jit.cpp and dali/array/gemm/cpu_gemm.cpp.
#ifndef DALI_B200_ORACLE_REF_BINDING_INCLUDES_H
#define DALI_B200_ORACLE_REF_BINDING_INCLUDES_H
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "dali_b200.h"
#endif
