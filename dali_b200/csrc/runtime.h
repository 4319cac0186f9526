// Internal runtime behind the C ABI: program registry, launch planning, NVRTC
// compile cache, per-device scratch arenas and the device memory pool.
#ifndef DALI_B200_CSRC_RUNTIME_H
#define DALI_B200_CSRC_RUNTIME_H

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "codegen.h"
#include "ir.h"

namespace dalib {

// thread-local error text
void set_error(const std::string& msg);
const std::string& get_error();

// A launch reduced to what the kernel needs: the variant compiled into the
// kernel plus the run-time parameter words and the grid.
struct LaunchPlan {
    Variant variant;
    std::vector<long long> words;   // kernel parameter block (scratch/counter filled at launch)
    unsigned grid_x = 1, grid_y = 1;
    size_t scratch_bytes = 0;       // cross-CTA exchange space this launch needs
    size_t counters = 0;            // ticket counters this launch needs
    bool empty = false;             // nothing to do (zero-sized space)
    std::string describe() const;
};

// Collapses the iteration space, classifies strides, picks skeleton + geometry.
// `strides[a]` may be null (contiguous).  Pointers are used for alignment only.
bool plan_launch(const Program& p, const int64_t* space, int rank,
                 void* const* array_data, const int64_t* offsets,
                 const int64_t* const* strides, int n_arrays,
                 const void* const* scalars, int n_scalars,
                 LaunchPlan* plan, std::string* err);

// NVRTC: CUDA C++ -> sm_100a cubin.  Works without a GPU.
bool nvrtc_compile(const std::string& source, const std::string& name,
                   std::vector<char>* cubin, std::string* log);

uint64_t fnv1a(const std::string& s, uint64_t seed = 1469598103934665603ull);

}  // namespace dalib
#endif
