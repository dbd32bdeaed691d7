// Test infrastructure. The reference's OpenBLAS glue (turbo_transformers/core/blas_openblas.cpp:20-41)
// needs Eigen, which is absent here. This file supplies the same two symbols with the same meaning:
// a batched sgemm that is a loop of sgemm calls, and an element-wise tanh.
#include <cmath>

#include "turbo_transformers/core/blas.h"

extern "C" {
void cblas_sgemm_batch(const CBLAS_ORDER order, const CBLAS_TRANSPOSE* ta, const CBLAS_TRANSPOSE* tb,
                       const blasint* m, const blasint* n, const blasint* k, const float* alpha,
                       const float** a, const blasint* lda, const float** b, const blasint* ldb,
                       const float* beta, float** c, const blasint* ldc, const blasint group_count,
                       const blasint* group_size) {
  int flat = 0;
  for (int g = 0; g < group_count; ++g) {
    for (int j = 0; j < group_size[g]; ++j, ++flat) {
      cblas_sgemm(order, ta[g], tb[g], m[g], n[g], k[g], alpha[g], a[flat], lda[g], b[flat], ldb[g], beta[g],
                  c[flat], ldc[g]);
    }
  }
}
void vsTanh(blasint n, const float* in, float* out) {
  for (int i = 0; i < n; ++i) out[i] = std::tanh(in[i]);
}
}
