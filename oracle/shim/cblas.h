/* Test-infrastructure stand-in for an OpenBLAS cblas.h (no BLAS headers on this image): the standard
 * CBLAS enums and the three entry points the reference's CPU path calls, resolved at link time by an
 * OpenBLAS shared object. */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef int blasint;
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, blasint m, blasint n, blasint k,
                 float alpha, const float* a, blasint lda, const float* b, blasint ldb, float beta, float* c,
                 blasint ldc);
void cblas_sscal(blasint n, float alpha, float* x, blasint incx);
void openblas_set_num_threads(int n);
#ifdef __cplusplus
}
#endif
