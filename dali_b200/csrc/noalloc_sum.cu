// dalib200_sum_f32_noalloc: all-axis fp32 sum that allocates nothing.
//
// For callers that are not allowed to allocate device memory when they call
// into this library: a real-time or interrupt-like host thread that must not
// take the allocator's locks or wait for the driver, an embedding whose memory
// budget is fixed at load time, code that runs after the process has handed
// all remaining device memory to something else.  The
// regular path (dalib200_launch on an all-axis reduction) takes its cross-CTA
// exchange space from an arena that grows with cudaMalloc on first use; this
// entry point keeps that space in a fixed array inside the library image
// instead, so every GPU that loads the library carries kScratchBytes of it
// until the process exits.
//
// Same algorithm as the generated all-axis reduction kernel: grid-stride
// partial sums with 128-bit loads, one partial per CTA written to the scratch
// array, a ticket counter, and the last CTA to arrive folds the partials in
// CTA order (the result does not depend on scheduling).
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

#include "../../include/dali_b200.h"
#include "runtime.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxCtas = 2048;                       // partials the scratch array can hold
constexpr int kLaunchCtas = 148 * 8;                 // CTAs launched at most: one full wave of 256-thread CTAs on 148 SMs
constexpr int kUnroll = 4;
constexpr size_t kPartialBytes = kMaxCtas * sizeof(float);
constexpr size_t kScratchBytes = kPartialBytes + 256;   // + one 256-byte line for the ticket counter
constexpr int kMaxDevices = 16;

// File-scope scratch: partial sums, then the ticket counter on its own line.
// In host code this name is only a handle for cudaGetSymbolAddress; kernels
// receive the device address obtained from it.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

__global__ void __launch_bounds__(kThreads)
sum_f32_noalloc_kernel(const float* __restrict__ x, long long n, float* out, float* partials, unsigned* counter) {
    __shared__ float warp_sums[kThreads / 32];
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    float acc = 0.0f;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) % 16 == 0);
    const long long n4 = vec_ok ? n / 4 : 0;
    const long long chunk = (long long)kThreads * kUnroll;
    for (long long base = (long long)blockIdx.x * chunk; base < n4; base += (long long)gridDim.x * chunk) {
        float4 q[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            long long i = base + (long long)u * kThreads + tid;
            q[u] = i < n4 ? reinterpret_cast<const float4*>(x)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) acc += (q[u].x + q[u].y) + (q[u].z + q[u].w);
    }
    // tail (and the whole array when x is not 16-byte aligned)
    for (long long i = n4 * 4 + (long long)blockIdx.x * kThreads + tid; i < n; i += (long long)gridDim.x * kThreads) acc += x[i];

    auto block_sum = [&](float v) {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
        if ((tid & 31) == 0) warp_sums[tid >> 5] = v;
        __syncthreads();
        float r = 0.0f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) r += warp_sums[w];
        return r;
    };
    float total = block_sum(acc);
    if (gridDim.x > 1) {
        if (tid == 0) {
            partials[blockIdx.x] = total;
            __threadfence();
            unsigned t = atomicInc(counter, gridDim.x - 1);   // wraps to 0 with the last arrival
            is_last = (t == gridDim.x - 1);
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        float v = 0.0f;
        for (unsigned b = tid; b < gridDim.x; b += kThreads) v += __ldcg(partials + b);
        __syncthreads();
        total = block_sum(v);
    }
    if (tid == 0) *out = total;
}

std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" int dalib200_sum_f32_noalloc(int device, void* stream, const float* x, int64_t n, float* out) {
    dalib::DeviceRestore restore_device;
    if (device < 0 || device >= kMaxDevices || device >= dalib200_device_count()) {
        dalib::set_error("dalib200_sum_f32_noalloc: device index out of range (call dalib200_init first)");
        return dalib200_device_count() == 0 ? DALIB200_ERR_NO_DEVICE : DALIB200_ERR_INVALID;
    }
    if (!x || !out || n < 0) {
        dalib::set_error("dalib200_sum_f32_noalloc: null pointer or negative size");
        return DALIB200_ERR_INVALID;
    }
    if (n > DALIB200_NOALLOC_MAX_ELEMENTS) {
        dalib::set_error("dalib200_sum_f32_noalloc: " + std::to_string((long long)n) + " elements exceed the fixed maximum of " +
                         std::to_string((long long)DALIB200_NOALLOC_MAX_ELEMENTS) +
                         " (2^31); use dalib200_launch, whose scratch grows on demand");
        return DALIB200_ERR_TOO_LARGE;
    }
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { dalib::set_error(std::string("cudaSetDevice: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    unsigned char* scratch = nullptr;
    {
        // once per device, with that device current: device address of the file-scope array
        std::lock_guard<std::mutex> g(g_mu);
        if (!g_scratch_addr[device]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                dalib::set_error(std::string("cudaGetSymbolAddress(noalloc scratch): ") + cudaGetErrorString(e));
                return DALIB200_ERR_CUDA;
            }
            g_scratch_addr[device] = static_cast<unsigned char*>(p);
        }
        scratch = g_scratch_addr[device];
    }
    float* partials = reinterpret_cast<float*>(scratch);
    unsigned* counter = reinterpret_cast<unsigned*>(scratch + kPartialBytes);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps what the previous call left: the ticket must start at zero (it does
    // after a completed call, but not after one that was torn down half way)
    e = cudaMemsetAsync(counter, 0, sizeof(unsigned), s);
    if (e != cudaSuccess) { dalib::set_error(std::string("cudaMemsetAsync: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    long long per_cta = (long long)kThreads * kUnroll * 4;
    long long ctas = (n + per_cta - 1) / per_cta;
    if (ctas < 1) ctas = 1;
    if (ctas > kLaunchCtas) ctas = kLaunchCtas;
    static_assert(kLaunchCtas <= kMaxCtas, "one partial per launched CTA must fit the scratch array");
    sum_f32_noalloc_kernel<<<(unsigned)ctas, kThreads, 0, s>>>(x, (long long)n, out, partials, counter);
    e = cudaGetLastError();
    if (e != cudaSuccess) { dalib::set_error(std::string("sum_f32_noalloc_kernel launch: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    return DALIB200_OK;
}
