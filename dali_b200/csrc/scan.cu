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
// coalesced; HBM bound: 2 * sizeof(T) bytes per element.  Rows shorter than a warp's tile go to
// groups of 1 .. 16 lanes (a [16M, 4] matrix keeps every lane busy); few, very long rows are cut
// into pieces that are scanned in two passes (piece totals, then the pieces), so that four rows
// of 16M elements still fill the machine: one more read of the input.
//
// inclusive: out[r][i] = x[r][0] (+) ... (+) x[r][i], out is [rows, cols]
// exclusive: out[r][0] = neutral element, out[r][i + 1] = inclusive[r][i], out is
//            [rows, cols + 1] (scan.cpp:9-15, 66-77)
// The neutral elements are the reference's (0, 1, lowest, max:
// dali/array/jit/reducer_kernels.h:10-54).
#include <cuda_runtime.h>

#include <cfloat>
#include <climits>
#include <algorithm>
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

// shuffles inside segments of w lanes (w a power of two up to 32)
template <typename T> __device__ T shfl_up(T v, int d, int w) { return __shfl_up_sync(0xffffffffu, v, d, w); }
template <> __device__ double shfl_up<double>(double v, int d, int w) {
    long long b = __double_as_longlong(v);
    int lo = __shfl_up_sync(0xffffffffu, (int)(b & 0xffffffffLL), d, w), hi = __shfl_up_sync(0xffffffffu, (int)(b >> 32), d, w);
    return __longlong_as_double(((long long)hi << 32) | (unsigned int)lo);
}
template <typename T> __device__ T shfl_idx(T v, int l, int w) { return __shfl_sync(0xffffffffu, v, l, w); }
template <> __device__ double shfl_idx<double>(double v, int l, int w) {
    long long b = __double_as_longlong(v);
    int lo = __shfl_sync(0xffffffffu, (int)(b & 0xffffffffLL), l, w), hi = __shfl_sync(0xffffffffu, (int)(b >> 32), l, w);
    return __longlong_as_double(((long long)hi << 32) | (unsigned int)lo);
}
template <typename T> __device__ T shfl_xor(T v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
template <> __device__ double shfl_xor<double>(double v, int m) {
    long long b = __double_as_longlong(v);
    int lo = __shfl_xor_sync(0xffffffffu, (int)(b & 0xffffffffLL), m), hi = __shfl_xor_sync(0xffffffffu, (int)(b >> 32), m);
    return __longlong_as_double(((long long)hi << 32) | (unsigned int)lo);
}

constexpr int kItems = 8;       // consecutive elements per thread and tile
constexpr int kThreads = 256;   // threads per CTA

// Op over all threads of the CTA (every thread gets the result); `sm` holds kThreads / 32 values
template <typename T, typename Op>
__device__ T block_fold(T v, T* sm) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = Op::apply(v, shfl_xor(v, m));
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    T all = Op::template init<T>();
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) all = Op::apply(all, sm[w]);
    __syncthreads();
    return all;
}

// G threads per row (1 .. 32, or kThreads); a CTA holds kThreads / G rows.
// VEC: rows start 16-byte aligned and row pitches keep that alignment (inclusive scans only: the
// exclusive output is shifted by one element).
// nchunks > 1 (G = kThreads only): a row is cut into nchunks pieces of `chunk` elements (a multiple of
// kThreads * kItems), one work item each; the running total a piece starts from is the fold of the totals of the
// pieces before it, which chunk_totals_kernel has left in `totals`.
template <typename T, typename Op, int G, bool VEC>
__global__ void __launch_bounds__(kThreads) scan_rows_kernel(const T* __restrict__ in, long long in_ld, T* __restrict__ out,
                                                             long long out_ld, long long rows, long long cols, int exclusive,
                                                             long long chunk, long long nchunks, const T* __restrict__ totals) {
    constexpr int kChunks = kItems * (int)sizeof(T) / 16;     // 128-bit pieces of a thread's elements
    constexpr int W = G < 32 ? G : 32;                        // lanes that share a row inside a warp
    __shared__ T warp_total[kThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = threadIdx.x % G;                       // position in the row's group
    const int gl = lane % W;                             // position in the group's part of the warp
    const long long rows_per_cta = kThreads / G;
    const long long items = rows * nchunks;              // (row, piece) pairs; nchunks = 1 unless G = kThreads
    for (long long item0 = (long long)blockIdx.x * rows_per_cta; item0 < items; item0 += (long long)gridDim.x * rows_per_cta) {
        const long long item = item0 + threadIdx.x / G;
        const bool live = item < items;                  // whole warps agree when G >= 32
        const long long row = live ? item / nchunks : 0, piece = live ? item % nchunks : 0;
        const long long begin = piece * chunk, end = (begin + chunk < cols) ? begin + chunk : cols;
        const T* x = in + row * in_ld;
        T* y = out + row * out_ld + (exclusive ? 1 : 0);
        T carry = Op::template init<T>();
        if (G == kThreads && nchunks > 1) {
            T part = Op::template init<T>();
            for (long long j = threadIdx.x; j < piece; j += kThreads) part = Op::apply(part, totals[row * nchunks + j]);
            carry = block_fold<T, Op>(part, warp_total);
        }
        if (live && exclusive && g == 0 && piece == 0) y[-1] = carry;
        for (long long base = begin; base < end; base += (long long)G * kItems) {
            const long long i0 = base + (long long)g * kItems;
            alignas(16) T v[kItems];
            // 128-bit pieces that lie inside the row go as one access each (a row of four floats is one piece), the
            // ragged rest element by element
            constexpr int kPer16 = 16 / (int)sizeof(T);
            if (VEC) {
#pragma unroll
                for (int q = 0; q < kChunks; ++q) {
                    if (live && i0 + (q + 1) * kPer16 <= end) {
                        reinterpret_cast<uint4*>(v)[q] = reinterpret_cast<const uint4*>(x + i0)[q];
                    } else {
#pragma unroll
                        for (int k = q * kPer16; k < (q + 1) * kPer16; ++k) v[k] = (live && i0 + k < end) ? x[i0 + k] : Op::template init<T>();
                    }
                }
            } else {
#pragma unroll
                for (int k = 0; k < kItems; ++k) v[k] = (live && i0 + k < end) ? x[i0 + k] : Op::template init<T>();
            }
#pragma unroll
            for (int k = 1; k < kItems; ++k) v[k] = Op::apply(v[k - 1], v[k]);
            // inclusive scan of the thread totals inside the group's lanes
            T tot = v[kItems - 1];
#pragma unroll
            for (int d = 1; d < W; d <<= 1) {
                const T o = shfl_up(tot, d, W);
                if (gl >= d) tot = Op::apply(o, tot);
            }
            T before = shfl_up(tot, 1, W);               // total of the lanes to the left
            if (gl == 0) before = Op::template init<T>();
            T tile_total = shfl_idx(tot, W - 1, W);
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
            if (VEC) {
#pragma unroll
                for (int q = 0; q < kChunks; ++q) {
                    if (live && i0 + (q + 1) * kPer16 <= end) {
                        reinterpret_cast<uint4*>(y + i0)[q] = reinterpret_cast<const uint4*>(v)[q];
                    } else {
#pragma unroll
                        for (int k = q * kPer16; k < (q + 1) * kPer16; ++k)
                            if (live && i0 + k < end) y[i0 + k] = v[k];
                    }
                }
            } else {
#pragma unroll
                for (int k = 0; k < kItems; ++k)
                    if (live && i0 + k < end) y[i0 + k] = v[k];
            }
            carry = Op::apply(carry, tile_total);
        }
    }
}

// totals[row * nchunks + piece] = Op over the piece's elements (first pass of the scan of few, very long rows)
template <typename T, typename Op, bool VEC>
__global__ void __launch_bounds__(kThreads) chunk_totals_kernel(const T* __restrict__ in, long long in_ld, long long rows, long long cols,
                                                                long long chunk, long long nchunks, T* __restrict__ totals) {
    constexpr int kPer16 = 16 / (int)sizeof(T);
    __shared__ T sm[kThreads / 32];
    for (long long item = blockIdx.x; item < rows * nchunks; item += gridDim.x) {
        const long long row = item / nchunks, piece = item % nchunks;
        const long long begin = piece * chunk, end = (begin + chunk < cols) ? begin + chunk : cols;
        const T* x = in + row * in_ld;
        T acc = Op::template init<T>();
        long long i = begin + (long long)threadIdx.x * kPer16;
        if (VEC) {
            for (; i + kPer16 <= end; i += (long long)kThreads * kPer16) {
                alignas(16) T v[kPer16];
                *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(x + i);
#pragma unroll
                for (int k = 0; k < kPer16; ++k) acc = Op::apply(acc, v[k]);
            }
            for (int k = 0; k < kPer16; ++k)
                if (i + k < end) acc = Op::apply(acc, x[i + k]);            // the ragged tail of the last piece
        } else {
            for (long long j = begin + threadIdx.x; j < end; j += kThreads) acc = Op::apply(acc, x[j]);
        }
        const T all = block_fold<T, Op>(acc, sm);
        if (threadIdx.x == 0) totals[item] = all;
    }
}

template <typename T, typename Op, int G>
void launch_rows(cudaStream_t stream, bool vec, long long ctas, const T* in, long long in_ld, T* out, long long out_ld, long long rows,
                 long long cols, int ex, long long chunk = 0, long long nchunks = 1, const T* totals = nullptr) {
    if (chunk == 0) chunk = cols;
    if (vec) scan_rows_kernel<T, Op, G, true><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, out, out_ld, rows, cols, ex, chunk, nchunks, totals);
    else scan_rows_kernel<T, Op, G, false><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, out, out_ld, rows, cols, ex, chunk, nchunks, totals);
}

template <typename T, typename Op>
cudaError_t launch_scan(int device, cudaStream_t stream, const T* in, long long in_ld, T* out, long long out_ld, long long rows,
                        long long cols, bool exclusive) {
    if (rows <= 0) return cudaSuccess;
    const long long per16 = 16 / (long long)sizeof(T);
    const bool in_vec = ((uintptr_t)in % 16 == 0) && in_ld % per16 == 0;
    const bool vec = !exclusive && in_vec && ((uintptr_t)out % 16 == 0) && out_ld % per16 == 0;
    const int ex = exclusive ? 1 : 0;
    const long long max_ctas = 148 * 16;
    if (cols <= 32 * kItems * 4) {
        // short rows: the smallest group of lanes whose one tile covers the row (a warp walks up to four tiles)
        int G = 1;
        while (G < 32 && (long long)G * kItems < cols) G <<= 1;
        const long long per = kThreads / G;
        const long long ctas = std::min((rows + per - 1) / per, max_ctas);
        switch (G) {
            case 1: launch_rows<T, Op, 1>(stream, vec, ctas, in, in_ld, out, out_ld, rows, cols, ex); break;
            case 2: launch_rows<T, Op, 2>(stream, vec, ctas, in, in_ld, out, out_ld, rows, cols, ex); break;
            case 4: launch_rows<T, Op, 4>(stream, vec, ctas, in, in_ld, out, out_ld, rows, cols, ex); break;
            case 8: launch_rows<T, Op, 8>(stream, vec, ctas, in, in_ld, out, out_ld, rows, cols, ex); break;
            case 16: launch_rows<T, Op, 16>(stream, vec, ctas, in, in_ld, out, out_ld, rows, cols, ex); break;
            default: launch_rows<T, Op, 32>(stream, vec, ctas, in, in_ld, out, out_ld, rows, cols, ex); break;
        }
        return cudaGetLastError();
    }
    // few, very long rows: cut every row into pieces so that the machine is full; pass 1 leaves each piece's total,
    // pass 2 scans the pieces, each starting from the fold of the totals before it (one more read of the input,
    // nothing waits on anything)
    const long long tile = (long long)kThreads * kItems;
    const long long want = 148 * 8;
    if (rows < want / 2 && cols >= 8 * tile) {
        long long nchunks = std::min((want + rows - 1) / rows, cols / (4 * tile));
        long long chunk = ((cols + nchunks - 1) / nchunks + tile - 1) / tile * tile;
        nchunks = (cols + chunk - 1) / chunk;
        if (nchunks > 1) {
            void* totals = nullptr;
            if (scratch_space(device, stream, (size_t)(rows * nchunks) * sizeof(T), &totals) != DALIB200_OK) return cudaErrorMemoryAllocation;
            const long long ctas = std::min(rows * nchunks, max_ctas);
            if (in_vec) chunk_totals_kernel<T, Op, true><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, rows, cols, chunk, nchunks, (T*)totals);
            else chunk_totals_kernel<T, Op, false><<<(unsigned)ctas, kThreads, 0, stream>>>(in, in_ld, rows, cols, chunk, nchunks, (T*)totals);
            launch_rows<T, Op, kThreads>(stream, vec, ctas, in, in_ld, out, out_ld, rows, cols, ex, chunk, nchunks, (const T*)totals);
            return cudaGetLastError();
        }
    }
    launch_rows<T, Op, kThreads>(stream, vec, std::min(rows, max_ctas), in, in_ld, out, out_ld, rows, cols, ex);
    return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch_op(int device, int op, cudaStream_t stream, const void* in, long long in_ld, void* out, long long out_ld, long long rows,
                        long long cols, bool exclusive) {
    const T* i = static_cast<const T*>(in);
    T* o = static_cast<T*>(out);
    switch (op) {
        case DALIB200_SCAN_SUM: return launch_scan<T, OpSum>(device, stream, i, in_ld, o, out_ld, rows, cols, exclusive);
        case DALIB200_SCAN_PROD: return launch_scan<T, OpProd>(device, stream, i, in_ld, o, out_ld, rows, cols, exclusive);
        case DALIB200_SCAN_MAX: return launch_scan<T, OpMax>(device, stream, i, in_ld, o, out_ld, rows, cols, exclusive);
        default: return launch_scan<T, OpMin>(device, stream, i, in_ld, o, out_ld, rows, cols, exclusive);
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
        case DALIB200_F32: e = dispatch_op<float>(device, op, s, in, in_row_stride, out, out_row_stride, rows, cols, !inclusive); break;
        case DALIB200_F64: e = dispatch_op<double>(device, op, s, in, in_row_stride, out, out_row_stride, rows, cols, !inclusive); break;
        case DALIB200_I32: e = dispatch_op<int>(device, op, s, in, in_row_stride, out, out_row_stride, rows, cols, !inclusive); break;
        default: set_error("dalib200_scan: dtype must be f32, f64 or i32"); return DALIB200_ERR_INVALID;
    }
    if (e != cudaSuccess) { set_error(std::string("dalib200_scan: ") + cudaGetErrorString(e)); return DALIB200_ERR_CUDA; }
    count_launch();
    return DALIB200_OK;
}
