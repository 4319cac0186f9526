// Splits fp32 operands for the 3xTF32 GEMM: hi keeps the 10 mantissa bits TF32
// carries (the low 13 bits cleared), lo = x - hi is exact in fp32.  The tensor
// cores then see hi without any further rounding, and
//   a.b ~= a_hi.b_hi + a_lo.b_hi + a_hi.b_lo
// is good to about 2^-21 relative to |a||b|, which is what fp32 parity with the
// reference's sgemm (1e-5) needs; one TF32 pass alone gives 1e-3.
#include <cuda_runtime.h>
#include <stdint.h>

#include "runtime.h"

namespace dalib {
// lo = x - hi, except for an infinite x: hi is then the infinity itself and inf - inf would turn every product with
// this element into NaN where an fp32 GEMM gives +-inf; a zero low part keeps inf . y = inf (and inf . 0 = NaN, as there).
__device__ __forceinline__ float tf32_lo(float v, float h) { return fabsf(h) == __int_as_float(0x7f800000) ? 0.0f : v - h; }


__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ x, long long rows, long long cols4, long long ld4, float4* __restrict__ hi,
                  float4* __restrict__ lo) {
    // rows x cols4 float4 groups; input row stride ld4 groups, outputs tight (cols4)
    const long long total = rows * cols4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols4, c = i - r * cols4;
        const float4 v = reinterpret_cast<const float4*>(x)[r * ld4 + c];
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = tf32_lo(v.x, h.x);
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = tf32_lo(v.y, h.y);
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = tf32_lo(v.z, h.z);
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = tf32_lo(v.w, h.w);
        hi[i] = h;
        lo[i] = l;
    }
}

// two operands of the same shape in one launch (blockIdx.y picks the operand): the x and h of a
// recurrent cell, which are split anew every step
struct SplitPair {
    const float* x[2];
    long long ld4[2];
    float4* hi[2];
    float4* lo[2];
};
__global__ void __launch_bounds__(256) split_tf32_pair_kernel(const SplitPair p, long long rows, long long cols4) {
    // launched as a programmatic dependent: wait for the kernel before this one, then let the GEMM that follows
    // start setting itself up (it waits for this grid to complete before it reads hi / lo)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int w = blockIdx.y;
    const long long total = rows * cols4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols4, c = i - r * cols4;
        const float4 v = reinterpret_cast<const float4*>(p.x[w])[r * p.ld4[w] + c];
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = tf32_lo(v.x, h.x);
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = tf32_lo(v.y, h.y);
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = tf32_lo(v.z, h.z);
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = tf32_lo(v.w, h.w);
        p.hi[w][i] = h;
        p.lo[w][i] = l;
    }
}

// same, writing the parts TRANSPOSED ([cols, rows], tight): 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256)
split_tf32_transpose_kernel(const float* __restrict__ x, long long rows, long long cols, long long ld, float* __restrict__ hi,
                            float* __restrict__ lo) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;           // 32 x 8
    const long long tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
    for (long long t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
        const long long r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long r = r0 + ty + 8 * i, c = c0 + tx;
            tile[ty + 8 * i][tx] = (r < rows && c < cols) ? x[r * ld + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long c = c0 + ty + 8 * i, r = r0 + tx;        // output row = input column
            if (c < cols && r < rows) {
                const float v = tile[tx][ty + 8 * i];
                const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
                hi[c * rows + r] = h;
                lo[c * rows + r] = tf32_lo(v, h);
            }
        }
        __syncthreads();
    }
}

// x: rows x cols (cols % 4 == 0, ld % 4 == 0, 16-byte aligned); hi / lo: tight, rows x cols or
// (transpose) cols x rows
cudaError_t split_tf32(cudaStream_t stream, const float* x, long long rows, long long cols, long long ld, bool transpose,
                       float* hi, float* lo) {
    if (transpose) {
        long long tiles = ((cols + 31) / 32) * ((rows + 31) / 32);
        if (tiles == 0) return cudaSuccess;
        if (tiles > 148 * 32) tiles = 148 * 32;
        split_tf32_transpose_kernel<<<(unsigned)tiles, 256, 0, stream>>>(x, rows, cols, ld, hi, lo);
        return cudaGetLastError();
    }
    const long long total = rows * (cols / 4);
    if (total == 0) return cudaSuccess;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    split_tf32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, rows, cols / 4, ld / 4, reinterpret_cast<float4*>(hi),
                                                            reinterpret_cast<float4*>(lo));
    return cudaGetLastError();
}

cudaError_t split_tf32_pair(cudaStream_t stream, const float* x0, const float* x1, long long rows, long long cols, long long ld0,
                            long long ld1, float* hi0, float* lo0, float* hi1, float* lo1) {
    const long long total = rows * (cols / 4);
    if (total == 0) return cudaSuccess;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    SplitPair p;
    p.x[0] = x0; p.x[1] = x1;
    p.ld4[0] = ld0 / 4; p.ld4[1] = ld1 / 4;
    p.hi[0] = reinterpret_cast<float4*>(hi0); p.hi[1] = reinterpret_cast<float4*>(hi1);
    p.lo[0] = reinterpret_cast<float4*>(lo0); p.lo[1] = reinterpret_cast<float4*>(lo1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks, 2);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    if (dependent_launch_enabled()) { cfg.attrs = &attr; cfg.numAttrs = 1; }
    return cudaLaunchKernelEx(&cfg, split_tf32_pair_kernel, p, rows, cols / 4);
}

}  // namespace dalib
