// Exact-precision GEMM on the CUDA cores (fp32 FMA accumulation) for the fp32 path and for the
// primitive MatMul / BatchMatMul entry points. The tensor-core GEMM lives in ttb_gemm_tc.cu.
#include "ttb_common.cuh"

using namespace ttb;

namespace {

// Tile shapes (256 threads each): 64 x 64 x 16 with 4 x 4 outputs per thread; 32 x 32 x 64 with 2 x 2 for problems whose
// 64 x 64 grid would leave most SMs idle (one 128-token request: 24 CTAs), where the long k step keeps 16 loads per thread
// in flight because there are too few CTAs to hide a load behind another CTA's arithmetic. Every output element sums its k terms in the same order in
// both, so the two give identical bits.

// C[b] = alpha * op(A[b]) * op(B[b]) + beta * C[b]; all row-major.
// op(A) is M x K: element (m,k) at A[m*K + k] or, transposed storage, A[k*M + m].
// op(B) is K x N: element (k,n) at B[k*N + n] or, transposed storage, B[n*K + k].
template <typename T, int BM, int BN, int TM, int TN, int BK>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, int a_trans, const T* __restrict__ B, int b_trans, T* __restrict__ C, int M,
                 int N, int K, float alpha, float beta, int64_t strideA, int64_t strideB, int64_t strideC) {
  constexpr int kPad = BM == 32 ? 1 : 4;  // odd row pitch: the 32 k values a warp stages for one row land in 32 banks
  __shared__ float As[BK][BM + kPad];
  __shared__ float Bs[BK][BN + kPad];
  const int batch = blockIdx.z;
  A += batch * strideA;
  B += batch * strideB;
  C += batch * strideC;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  static_assert((BM / TM) * (BN / TN) == 256, "256 threads per tile");
  constexpr int EA = BM * BK / 256, EB = BN * BK / 256;  // tile elements per thread
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);  // thread owns rows ty*TM.., cols tx*TN..
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // The next k block is fetched into registers while the current one is multiplied out of shared memory, so a global
  // load's latency overlaps the arithmetic instead of adding to every step of the k loop.
  float ra[EA], rb[EB];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int e = 0; e < EA; ++e) {
      const int idx = tid + e * 256;
      int m, k;
      if (a_trans) { m = idx % BM; k = idx / BM; } else { k = idx % BK; m = idx / BK; }
      const int gm = m0 + m, gk = k0 + k;
      ra[e] = (gm < M && gk < K) ? to_f(a_trans ? A[(int64_t)gk * M + gm] : A[(int64_t)gm * K + gk]) : 0.f;
    }
#pragma unroll
    for (int e = 0; e < EB; ++e) {
      const int idx = tid + e * 256;
      int n, k;
      if (b_trans) { k = idx % BK; n = idx / BK; } else { n = idx % BN; k = idx / BN; }
      const int gn = n0 + n, gk = k0 + k;
      rb[e] = (gn < N && gk < K) ? to_f(b_trans ? B[(int64_t)gn * K + gk] : B[(int64_t)gk * N + gn]) : 0.f;
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int e = 0; e < EA; ++e) {
      const int idx = tid + e * 256;
      if (a_trans) As[idx / BM][idx % BM] = ra[e]; else As[idx % BK][idx / BK] = ra[e];
    }
#pragma unroll
    for (int e = 0; e < EB; ++e) {
      const int idx = tid + e * 256;
      if (b_trans) Bs[idx % BK][idx / BK] = rb[e]; else Bs[idx / BN][idx % BN] = rb[e];
    }
  };

  if (K > 0) fetch(0);
  for (int k0 = 0; k0 < K; k0 += BK) {
    stage();
    __syncthreads();
    if (k0 + BK < K) fetch(k0 + BK);
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
  const bool small = ((M + 63) / 64) * ((N + 63) / 64) * batch < 2ll * ctx->sm_count;  // too few 64 x 64 tiles to fill the GPU
  const int bm = small ? 32 : 64;
  const int64_t gy = (M + bm - 1) / bm, gx = (N + bm - 1) / bm;
  TTB_REQUIRE(ctx, gy <= 65535, "%s: M too large for this kernel", what);
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (int)(batch - b0 < 65535 ? batch - b0 : 65535);
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)nb);
    if (small) {
      TTB_DISPATCH_FLOAT(ctx, dtype, T,
                         (gemm_simt_kernel<T, 32, 32, 2, 2, 64><<<grid, 256, 0, ctx->stream>>>((const T*)A + b0 * M * K, a_trans, (const T*)B + b0 * K * N,
                                                                                          b_trans, (T*)C + b0 * M * N, (int)M, (int)N, (int)K,
                                                                                          alpha, beta, M * K, K * N, M * N)));
    } else {
      TTB_DISPATCH_FLOAT(ctx, dtype, T,
                         (gemm_simt_kernel<T, 64, 64, 4, 4, 16><<<grid, 256, 0, ctx->stream>>>((const T*)A + b0 * M * K, a_trans, (const T*)B + b0 * K * N,
                                                                                          b_trans, (T*)C + b0 * M * N, (int)M, (int)N, (int)K,
                                                                                          alpha, beta, M * K, K * N, M * N)));
    }
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
