// General-purpose GEMM on CUDA cores for every layout and dtype the front end
// can hand over (strided, transposed, int32, fp64, tiny or ragged shapes).
// The tensor-core path (gemm_sm100.cu) takes the large aligned fp32 / bf16
// problems; this kernel is the one that is always applicable, in place of the
// reference's naive int kernel (dali/array/gemm/cublas_gemm.cu:62-108, which
// is launched with a single 16x16 block) and of cuBLAS for odd layouts.
#include <cuda_runtime.h>
#include <stdint.h>

namespace dalib {

template <typename T, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(int64_t m, int64_t n, int64_t k, const T* __restrict__ a, int64_t ars, int64_t acs,
                 const T* __restrict__ b, int64_t brs, int64_t bcs, T* c, int64_t crs, int64_t ccs, T alpha, T beta) {
    __shared__ T sa[BK][BM + 1];
    __shared__ T sb[BK][BN + 1];
    const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
    const int nthreads = (BM / TM) * (BN / TN);
    const int64_t row0 = (int64_t)blockIdx.y * BM, col0 = (int64_t)blockIdx.x * BN;
    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = (T)0;
    for (int64_t k0 = 0; k0 < k; k0 += BK) {
        for (int idx = threadIdx.x; idx < BM * BK; idx += nthreads) {
            // consecutive threads walk whichever of A's two dims is the contiguous one
            int r, kk;
            if (acs == 1) { kk = idx % BK; r = idx / BK; } else { r = idx % BM; kk = idx / BM; }
            int64_t gr = row0 + r, gk = k0 + kk;
            sa[kk][r] = (gr < m && gk < k) ? a[gr * ars + gk * acs] : (T)0;
        }
        for (int idx = threadIdx.x; idx < BN * BK; idx += nthreads) {
            int cidx, kk;
            if (bcs == 1) { cidx = idx % BN; kk = idx / BN; } else { kk = idx % BK; cidx = idx / BK; }
            int64_t gc = col0 + cidx, gk = k0 + kk;
            sb[kk][cidx] = (gc < n && gk < k) ? b[gk * brs + gc * bcs] : (T)0;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            T ra[TM], rb[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ra[i] = sa[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) rb[j] = sb[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] += ra[i] * rb[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int64_t gr = row0 + ty * TM + i;
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int64_t gc = col0 + tx * TN + j;
            if (gc >= n) continue;
            T* p = c + gr * crs + gc * ccs;
            T v = alpha * acc[i][j];
            if (beta != (T)0) v += beta * *p;
            *p = v;
        }
    }
}

template <typename T>
static cudaError_t launch_simt(cudaStream_t stream, int64_t m, int64_t n, int64_t k, const void* a, int64_t ars,
                               int64_t acs, const void* b, int64_t brs, int64_t bcs, void* c, int64_t crs, int64_t ccs,
                               double alpha, double beta) {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    dim3 grid((unsigned)((n + BN - 1) / BN), (unsigned)((m + BM - 1) / BM));
    gemm_simt_kernel<T, BM, BN, BK, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, stream>>>(
        m, n, k, (const T*)a, ars, acs, (const T*)b, brs, bcs, (T*)c, crs, ccs, (T)alpha, (T)beta);
    return cudaGetLastError();
}

// dtype: 0 float, 1 double, 2 int32
cudaError_t gemm_simt(cudaStream_t stream, int dtype, int64_t m, int64_t n, int64_t k, const void* a, int64_t ars,
                      int64_t acs, const void* b, int64_t brs, int64_t bcs, void* c, int64_t crs, int64_t ccs,
                      double alpha, double beta) {
    if (dtype == 0) return launch_simt<float>(stream, m, n, k, a, ars, acs, b, brs, bcs, c, crs, ccs, alpha, beta);
    if (dtype == 1) return launch_simt<double>(stream, m, n, k, a, ars, acs, b, brs, bcs, c, crs, ccs, alpha, beta);
    return launch_simt<int>(stream, m, n, k, a, ars, acs, b, brs, bcs, c, crs, ccs, alpha, beta);
}

}  // namespace dalib
