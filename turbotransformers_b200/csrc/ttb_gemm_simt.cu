// Exact-precision GEMM on the CUDA cores (fp32 FMA accumulation) for the fp32 path and for the
// primitive MatMul / BatchMatMul entry points. The tensor-core GEMM lives in ttb_gemm_tc.cu.
#include "ttb_common.cuh"

using namespace ttb;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

// C[b] = alpha * op(A[b]) * op(B[b]) + beta * C[b]; all row-major.
// op(A) is M x K: element (m,k) at A[m*K + k] or, transposed storage, A[k*M + m].
// op(B) is K x N: element (k,n) at B[k*N + n] or, transposed storage, B[n*K + k].
template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, int a_trans, const T* __restrict__ B, int b_trans, T* __restrict__ C, int M,
                 int N, int K, float alpha, float beta, int64_t strideA, int64_t strideB, int64_t strideC) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int batch = blockIdx.z;
  A += batch * strideA;
  B += batch * strideB;
  C += batch * strideC;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // thread owns rows ty*4.., cols tx*4..
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // A tile: BM x BK = 1024 elements, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      int m, k;
      if (a_trans) { m = idx % BM; k = idx / BM; } else { k = idx % BK; m = idx / BK; }
      const int gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < M && gk < K) v = to_f(a_trans ? A[(int64_t)gk * M + gm] : A[(int64_t)gm * K + gk]);
      As[k][m] = v;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      int n, k;
      if (b_trans) { k = idx % BK; n = idx / BK; } else { n = idx % BN; k = idx / BN; }
      const int gn = n0 + n, gk = k0 + k;
      float v = 0.f;
      if (gn < N && gk < K) v = to_f(b_trans ? B[(int64_t)gn * K + gk] : B[(int64_t)gk * N + gn]);
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float r = alpha * acc[i][j];
      if (beta != 0.f) r += beta * to_f(C[(int64_t)gm * N + gn]);
      C[(int64_t)gm * N + gn] = from_f<T>(r);
    }
  }
}

int run(ttb_ctx* ctx, int dtype, const void* A, int a_trans, const void* B, int b_trans, int64_t batch, int64_t M,
        int64_t N, int64_t K, float alpha, float beta, void* C, const char* what) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, batch >= 0 && M >= 0 && N >= 0 && K >= 0, "%s: negative shape", what);
  TTB_REQUIRE(ctx, M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "%s: dimension too large", what);
  if (batch * M * N == 0) return TTB_OK;
  TTB_REQUIRE(ctx, C && (K == 0 || (A && B)), "%s: null pointer", what);
  DeviceGuard g(ctx->device);
  const int64_t gy = (M + BM - 1) / BM, gx = (N + BN - 1) / BN;
  TTB_REQUIRE(ctx, gy <= 65535, "%s: M too large for this kernel", what);
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (int)(batch - b0 < 65535 ? batch - b0 : 65535);
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)nb);
    TTB_DISPATCH_FLOAT(ctx, dtype, T,
                       gemm_simt_kernel<T><<<grid, 256, 0, ctx->stream>>>((const T*)A + b0 * M * K, a_trans, (const T*)B + b0 * K * N,
                                                                         b_trans, (T*)C + b0 * M * N, (int)M, (int)N, (int)K, alpha,
                                                                         beta, M * K, K * N, M * N));
    int s = launched(ctx, what);
    if (s) return s;
  }
  return TTB_OK;
}

}  // namespace

extern "C" int ttb_matmul(ttb_ctx* ctx, int dtype, const void* A, int a_trans, const void* B, int b_trans, int64_t M,
                          int64_t N, int64_t K, float alpha, float beta, void* C) {
  return run(ctx, dtype, A, a_trans, B, b_trans, 1, M, N, K, alpha, beta, C, "matmul");
}

extern "C" int ttb_batch_matmul(ttb_ctx* ctx, int dtype, const void* A, int a_trans, const void* B, int b_trans,
                                int64_t batch, int64_t M, int64_t N, int64_t K, float alpha, float beta, void* C) {
  return run(ctx, dtype, A, a_trans, B, b_trans, batch, M, N, K, alpha, beta, C, "batch_matmul");
}
