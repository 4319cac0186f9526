/* Test infrastructure only: the two CBLAS entry points the reference's CPU
 * gemm calls (dali/array/gemm/cpu_gemm.cpp:60-78).  Resolved at link time by
 * an OpenBLAS found on the machine, else by mini_cblas.c beside this file. */
#ifndef DALI_B200_ORACLE_CBLAS_SHIM_H
#define DALI_B200_ORACLE_CBLAS_SHIM_H
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb,
                 int m, int n, int k, float alpha, const float* a, int lda,
                 const float* b, int ldb, float beta, float* c, int ldc);
void cblas_dgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb,
                 int m, int n, int k, double alpha, const double* a, int lda,
                 const double* b, int ldb, double beta, double* c, int ldc);
#endif
