/* Test infrastructure only: fallback sgemm/dgemm for the reference build when
 * no OpenBLAS is found.  Column-major, cache-blocked, OpenMP over column
 * panels (single-threaded when built without OpenMP); accumulates each dot product in the operand type like a plain BLAS. */
#include "cblas.h"
#include <stddef.h>

#define MINI_GEMM(NAME, T)                                                                 \
void NAME(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb,        \
          int m, int n, int k, T alpha, const T* a, int lda, const T* b, int ldb,          \
          T beta, T* c, int ldc) {                                                         \
    if (order == CblasRowMajor) { /* C^T = B^T A^T in column-major */                      \
        NAME(CblasColMajor, tb, ta, n, m, k, alpha, b, ldb, a, lda, beta, c, ldc);         \
        return;                                                                            \
    }                                                                                      \
    const int BK = 256;                                                                    \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int j = 0; j < n; ++j) {                                                          \
        T* cj = c + (size_t)j * ldc;                                                       \
        for (int i = 0; i < m; ++i) cj[i] = (beta == (T)0) ? (T)0 : beta * cj[i];          \
        for (int p0 = 0; p0 < k; p0 += BK) {                                               \
            int p1 = p0 + BK < k ? p0 + BK : k;                                            \
            for (int p = p0; p < p1; ++p) {                                                \
                T bv = alpha * (tb == CblasNoTrans ? b[(size_t)j * ldb + p]                \
                                                   : b[(size_t)p * ldb + j]);             \
                if (ta == CblasNoTrans) {                                                  \
                    const T* ap = a + (size_t)p * lda;                                     \
                    for (int i = 0; i < m; ++i) cj[i] += ap[i] * bv;                       \
                } else {                                                                   \
                    for (int i = 0; i < m; ++i) cj[i] += a[(size_t)i * lda + p] * bv;      \
                }                                                                          \
            }                                                                              \
        }                                                                                  \
    }                                                                                      \
}
MINI_GEMM(cblas_sgemm, float)
MINI_GEMM(cblas_dgemm, double)
