// Running reduction (cumsum / cumprod / running max / min) along the rows of a
// [rows, cols] matrix: dalib200_scan.
//
// Replaces the reference's AxisScan kernels (dali/array/op/scan.cpp:47-180):
// its CPU body walks a row left to right, its GPU body gives one block per row
// and a Hillis-Steele pass over shared memory.  Here a row is owned by a group of
// G threads (a warp for short rows, a 256-thread CTA for long ones) that walks
// it in tiles of 8 G elements: every thread scans its 8 consecutive elements
// (128-bit loads and stores when rows are 16-byte aligned) in registers, thread
// totals are scanned with warp shuffles (and across the warps of a CTA through 8
// words of shared memory), and the running total of the tiles before is carried
// in a register.  One read and one write of the matrix, both
// coalesced; HBM bound: 2 * sizeof(T) bytes per element.
//
// inclusive: out[r][i] = x[r][0] (+) ... (+) x[r][i], out is [rows, cols]
// exclusive: out[r][0] = neutral element, out[r][i + 1] = inclusive[r][i], out is
//            [rows, cols + 1] (scan.cpp:9-15, 66-77)
// The neutral elements are the reference's (0, 1, lowest, max:
// dali/array/jit/reducer_kernels.h:10-54).
#include <cuda_runtime.h>

#include <cfloat>
#include <climits>
#include <cstdint>

#include "../../include/dali_b200.h"
#include "runtime.h"

namespace dalib {
namespace {

template <typename T> struct Limits;
template <> struct Limits<float> { static __device__ float lo() { return -FLT_MAX; } static __device__ float hi() { return FLT_MAX; } };
template <> struct Limits<double> { static __device__ double lo() { return -DBL_MAX; } static __device__ double hi() { return DBL_MAX; } };
template <> struct Limits<int> { static __device__ int lo() { return INT_MIN; } static __device__ int hi() { return INT_MAX; } };

struct OpSum { template <typename T> static __device__ T init() { return (T)0; } template <typename T> static __device__ T apply(T a, T b) { return a + b; } };
struct OpProd { template <typename T> static __device__ T init() { return (T)1; } template <typename T> static __device__ T apply(T a, T b) { return a * b; } };
struct OpMax { template <typename T> static __device__ T init() { return Limits<T>::lo(); } template <typename T> static __device__ T apply(T a, T b) { return a > b ? a : b; } };
struct OpMin { template <typename T> static __device__ T init() { return Limits<T>::hi(); } template <typename T> static __device__ T apply(T a, T b) { return a < b ? a : b; } };

template <typename T> __device__ T shfl_up(T v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
template <> __device__ double shfl_up<double>(double v, int d) {
    long long b = __double_as_longlong(v);
    int lo = __shfl_up_sync(0xffffffffu, (int)(b & 0xffffffffLL), d), hi = __shfl_up_sync(0xffffffffu, (int)(b >> 32), d);
    return __longlong_as_double(((long long)hi << 32) | (unsigned int)lo);
}
template <typename T> __device__ T shfl_idx(T v, int l) { return __shfl_sync(0xffffffffu, v, l); }
template <> __device__ double shfl_idx<double>(double v, int l) {
    long long b = __double_as_longlong(v);
    int lo = __shfl_sync(0xffffffffu, (int)(b & 0xffffffffLL), l), hi = __shfl_sync(0xffffffffu, (int)(b >> 32), l);
    return __longlong_as_double(((long long)hi << 32) | (unsigned int)lo);
}

constexpr int kItems = 8;       // consecutive elements per thread and tile
constexpr int kThreads = 256;   // threads per CTA

// G threads per row (32 or kThreads); a CTA holds kThreads / G rows
// VEC: rows start 16-byte aligned and row pitches keep that alignment (inclusive scans only: the
// exclusive output is shifted by one element)
template <typename T, typename Op, int G, bool VEC>
__global__ void __launch_bounds__(kThreads) scan_rows_kernel(const T* __restrict__ in, long long in_ld, T* __restrict__ out,
                                                             long long out_ld, long long rows, long long cols, int exclusive) {
    constexpr int kChunks = kItems * (int)sizeof(T) / 16;     // 128-bit pieces of a thread's elements
    __shared__ T warp_total[kThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = threadIdx.x % G;                       // position in the row's group
    const long long rows_per_cta = kThreads / G;
    for (long long row0 = (long long)blockIdx.x * rows_per_cta; row0 < rows; row0 += (long long)gridDim.x * rows_per_cta) {
        const long long row = row0 + threadIdx.x / G;
        const bool live = row < rows;                    // whole warps agree when G >= 32
        const T* x = in + (live ? row : 0) * in_ld;
        T* y = out + (live ? row : 0) * out_ld + (exclusive ? 1 : 0);
        T carry = Op::template init<T>();
        if (live && exclusive && g == 0) y[-1] = carry;
        for (long long base = 0; base < cols; base += (long long)G * kItems) {
            const long long i0 = base + (long long)g * kItems;
            alignas(16) T v[kItems];
            const bool whole = live && i0 + kItems <= cols;
            if (VEC && whole) {
#pragma unroll
                for (int q = 0; q < kChunks; ++q) reinterpret_cast<uint4*>(v)[q] = reinterpret_cast<const uint4*>(x + i0)[q];
            } else {
#pragma unroll
                for (int k = 0; k < kItems; ++k) v[k] = (live && i0 + k < cols) ? x[i0 + k] : Op::template init<T>();
            }
#pragma unroll
            for (int k = 1; k < kItems; ++k) v[k] = Op::apply(v[k - 1], v[k]);
            // inclusive scan of the thread totals inside the warp
            T tot = v[kItems - 1];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const T o = shfl_up(tot, d);
                if (lane >= d) tot = Op::apply(o, tot);
            }
            T before = shfl_up(tot, 1);                  // total of the lanes to the left
            if (lane == 0) before = Op::template init<T>();
            T tile_total = shfl_idx(tot, 31);
            if (G > 32) {
                // across the warps of the CTA (one row per CTA)
                if (lane == 31) warp_total[warp] = tot;
                __syncthreads();
                T left = Op::template init<T>(), all = Op::template init<T>();
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w) {
                    const T t = warp_total[w];
                    if (w < warp) left = Op::apply(left, t);
                    all = Op::apply(all, t);
                }
                __syncthreads();
                before = Op::apply(left, before);
                tile_total = all;
            }
            const T offset = Op::apply(carry, before);
#pragma unroll
            for (int k = 0; k < kItems; ++k) v[k] = Op::apply(offset, v[k]);
            if (VEC && whole) {
#pragma unroll
                for (int q = 0; q < kChunks; ++q) reinterpret_cast<uint4*>(y + i0)[q] = reinterpret_cast<const uint4*>(v)[q];
            } else {
#pragma unroll
                for (int k = 0; k < kItems; ++k)
                    if (live && i0 + k < cols) y[i0 + k] = v[k];
            }
            carry = Op::apply(carry, tile_total);
        }
    }
}

template <typename T, typename Op>
cudaError_t launch_scan(cudaStream_t stream, const T* in, long long in_ld, T* out, long long out_ld, long long rows, long long cols,
                        bool exclusive) {
    if (rows <= 0) return cudaSuccess;
    const long long per16 = 16 / (long long)sizeof(T);
    const bool vec = !exclusive && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && in_ld % per16 == 0 && out_ld % per16 == 0;
    const int ex = exclusive ? 1 : 0;
    if (cols <= 32 * kItems * 4) {
        const long long per = kThreads / 32;
        long long ctas = (rows + per - 1) / per;
        if (ctas > 148 * 16) ctas = 148 * 16;
        if (vec) scan_rows_kernel<T, Op, 32, true><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, out, out_ld, rows, cols, ex);
        else scan_rows_kernel<T, Op, 32, false><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, out, out_ld, rows, cols, ex);
    } else {
        long long ctas = rows > 148 * 16 ? 148 * 16 : rows;
        if (vec) scan_rows_kernel<T, Op, kThreads, true><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, out, out_ld, rows, cols, ex);
        else scan_rows_kernel<T, Op, kThreads, false><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, out, out_ld, rows, cols, ex);
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch_op(int op, cudaStream_t stream, const void* in, long long in_ld, void* out, long long out_ld, long long rows,
                        long long cols, bool exclusive) {
    const T* i = static_cast<const T*>(in);
    T* o = static_cast<T*>(out);
    switch (op) {
        case DALIB200_SCAN_SUM: return launch_scan<T, OpSum>(stream, i, in_ld, o, out_ld, rows, cols, exclusive);
        case DALIB200_SCAN_PROD: return launch_scan<T, OpProd>(stream, i, in_ld, o, out_ld, rows, cols, exclusive);
        case DALIB200_SCAN_MAX: return launch_scan<T, OpMax>(stream, i, in_ld, o, out_ld, rows, cols, exclusive);
        default: return launch_scan<T, OpMin>(stream, i, in_ld, o, out_ld, rows, cols, exclusive);
    }
}

}  // namespace
}  // namespace dalib

using namespace dalib;

extern "C" int dalib200_scan(int device, void* stream, int dtype, int op, int inclusive, int64_t rows, int64_t cols, const void* in,
                             int64_t in_row_stride, void* out, int64_t out_row_stride) {
    DeviceRestore restore_device;
    int ord = device_ordinal(device);
    if (ord < 0) { set_error("device index out of range"); return dalib200_device_count() ? DALIB200_ERR_INVALID : DALIB200_ERR_NO_DEVICE; }
    if (op < DALIB200_SCAN_SUM || op > DALIB200_SCAN_MIN || rows < 0 || cols < 0 || (rows > 0 && (!in && cols > 0)) || (rows > 0 && !out)) {
        set_error("dalib200_scan: bad argument");
        return DALIB200_ERR_INVALID;
    }
    if (rows == 0 || (cols == 0 && inclusive)) return DALIB200_OK;
    cudaSetDevice(ord);
    cudaError_t e;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
        case DALIB200_F32: e = dispatch_op<float>(op, s, in, in_row_stride, out, out_row_stride, rows, cols, !inclusive); break;
        case DALIB200_F64: e = dispatch_op<double>(op, s, in, in_row_stride, out, out_row_stride, rows, cols, !inclusive); break;
        case DALIB200_I32: e = dispatch_op<int>(op, s, in, in_row_stride, out, out_row_stride, rows, cols, !inclusive); break;
        default: set_error("dalib200_scan: dtype must be f32, f64 or i32"); return DALIB200_ERR_INVALID;
    }
    if (e != cudaSuccess) { set_error(std::string("dalib200_scan: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    count_launch();
    return DALIB200_OK;
}
