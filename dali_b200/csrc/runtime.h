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
    unsigned cluster = 0;           // CTAs per thread-block cluster (0 / 1: none)
    unsigned smem_bytes = 0;        // dynamic shared memory (the staged row variant's rings)
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
std::string nvrtc_defines_text();      // DALI_B200_DEFINES: macros handed to every generated kernel; part of the cache keys
bool nvrtc_compile(const std::string& source, const std::string& name,
                   std::vector<char>* cubin, std::string* log);

uint64_t fnv1a(const std::string& s, uint64_t seed = 1469598103934665603ull);

// Entry points select the device they work on with cudaSetDevice; this puts the caller's
// current device back when the entry point returns (a caller with several GPUs in one
// process, or torch with its own notion of the current device, must not see it move).
struct DeviceRestore {
    int prev;
    DeviceRestore();
    ~DeviceRestore();
};

// ---- services of runtime.cc for the other translation units ------------------------
// Copy of the program registered under `hash` (false if unknown).
bool find_program(uint64_t hash, Program* out);
// The device prelude text (functors, reducers) that precedes every generated kernel.
const char* device_prelude();
// Compiles (memory -> disk -> NVRTC) the kernel identified by `key`; `make_source` is
// only called on a miss.  With device >= 0 also loads it there and returns the function
// handle (a CUfunction) in *function.  Returns a dalib200_status.
typedef bool (*SourceFn)(void* ctx, std::string* source, std::string* err);
int acquire_kernel(int device, const std::string& key, const char* entry_name, SourceFn make_source, void* ctx,
                   void** function, size_t* cubin_size);
// cuLaunchKernel / cuFuncSetAttribute(max dynamic shared memory) on the bound device.
// dependent = true: programmatic dependent launch -- the kernel may start while its predecessor in the stream
// is still finishing and must itself execute griddepcontrol.wait before it touches global memory.
int launch_function(int device, void* function, unsigned gx, unsigned gy, unsigned threads, unsigned smem_bytes,
                    void* stream, void** params, bool dependent = false);
// DALI_B200_PDL != 0 (default on): kernels that are written for it are launched as programmatic dependents
bool dependent_launch_enabled();
// Driver entry point by name (nullptr if unavailable).
void* driver_entry(const char* name);
int device_ordinal(int device);            // CUDA ordinal of bound device, -1 if not bound
// At least `bytes` of the cross-CTA exchange space of (device, stream): the space generated kernels use for their
// partial results, valid until the next launch on that stream that asks for space.  Returns a dalib200_status.
int scratch_space(int device, void* stream, size_t bytes, void** out);
void count_launch();
// Device address of the peer table of the communicator's rank on `device` (comm.cc), nullptr without one.
const void* comm_peer_table(int device);
// One int per device that tensor-core kernels raise when a bounded wait expires.
int* gemm_error_word(int device);
// Remembers, per thread, which GEMM kernel served the last call (dalib200_last_gemm_kernel).
void note_gemm_kernel(const std::string& name);

}  // namespace dalib
#endif
