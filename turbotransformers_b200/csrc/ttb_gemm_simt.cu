// Exact-precision GEMM on the CUDA cores (fp32 FMA accumulation) for the fp32 path and for the
// primitive MatMul / BatchMatMul entry points. The tensor-core GEMM lives in ttb_gemm_tc.cu.
#include "ttb_common.cuh"

#include <algorithm>
#include <cstdint>
#include <type_traits>

using namespace ttb;

namespace {

// Tile shapes (256 threads each): 128 x 128 x 16 with 8 x 8 outputs per thread (gemm_simt_large_kernel below) for problems
// with at least two waves of such tiles; 64 x 64 x 16 with 4 x 4; 32 x 32 x 64 with 2 x 2 for problems whose
// 64 x 64 grid would leave most SMs idle (one 128-token request: 24 CTAs), where the long k step keeps 16 loads per thread
// in flight because there are too few CTAs to hide a load behind another CTA's arithmetic. Every output element sums its k terms in the same order in
// all of them, so they give identical bits; only the split-K path (small problems with a long k, see run()) adds partial
// sums of k slices instead, still in a fixed order.

// C[b] = alpha * op(A[b]) * op(B[b]) + beta * C[b]; all row-major.
// op(A) is M x K: element (m,k) at A[m*K + k] or, transposed storage, A[k*M + m].
// op(B) is K x N: element (k,n) at B[k*N + n] or, transposed storage, B[n*K + k].
template <typename T, int BM, int BN, int TM, int TN, int BK>
__global__ void __launch_bounds__(256, 2)
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
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  // Rows and columns a thread owns: TM (TN) consecutive ones, or, for 8, two groups of 4 half a tile apart, so that the
  // 16-byte shared-memory reads of neighbouring threads are contiguous (no bank conflicts).
  auto row_of = [&](int i) { return TM == 8 ? (i / 4) * (BM / 2) + ty * 4 + (i % 4) : ty * TM + i; };
  auto col_of = [&](int j) { return TN == 8 ? (j / 4) * (BN / 2) + tx * 4 + (j % 4) : tx * TN + j; };
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
      for (int i = 0; i < TM; ++i) a[i] = As[k][row_of(i)];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[k][col_of(j)];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + row_of(i);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + col_of(j);
      if (gn >= N) continue;
      float r = alpha * acc[i][j];
      if (beta != 0.f) r += beta * to_f(C[(int64_t)gm * N + gn]);
      C[(int64_t)gm * N + gn] = from_f<T>(r);
    }
  }
}


// ---- 128 x 128 x 16 and 64 x 128 x 16 tiles for large and medium problems ---------------------------------------------
// 256 threads, 8 x 8 outputs per thread as 2 x 2 groups of 4 x 4 half a tile apart (4 x 8 as 1 x 2 groups for the 64-row
// tile), so a k step is four (three) 16-byte shared-memory reads, contiguous across neighbouring threads, for 64 (32) FMAs. Shared memory is double-buffered (one barrier per
// k block) and the next k block travels global -> registers while the current one is multiplied. fp32 operands whose rows
// are 16-byte aligned are fetched as float4; tiles on a ragged edge and other types take checked scalar loads into the
// same register slots. Every output still sums its k terms in increasing k with one FMA each: same bits as the tiles above.
constexpr int LBN = 128, LBK = 16;

template <typename T>
__device__ __forceinline__ float4 fetch4(const T* __restrict__ P, bool vec, bool inside, int r, int k, int R, int K, int k_end,
                                         bool k_major) {
  // Four consecutive elements of an operand with R rows and K columns, zero at rows >= R and at k >= k_end. k_major: storage
  // is P[r * K + k] and the four run along k; otherwise storage is P[k * R + r] and the four run along r.
  if constexpr (std::is_same<T, float>::value) {
    if (vec && inside) {
      const float* q = k_major ? P + (int64_t)r * K + k : P + (int64_t)k * R + r;
      return *reinterpret_cast<const float4*>(q);
    }
  }
  float v[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int rr = k_major ? r : r + c, kk = k_major ? k + c : k;
    v[c] = (rr < R && kk < k_end) ? to_f(k_major ? P[(int64_t)rr * K + kk] : P[(int64_t)kk * R + rr]) : 0.f;
  }
  return make_float4(v[0], v[1], v[2], v[3]);
}

template <typename T, int LBM>
__global__ void __launch_bounds__(256, LBM == 64 ? 3 : 2)
gemm_simt_large_kernel(const T* __restrict__ A, int a_trans, const T* __restrict__ B, int b_trans, T* __restrict__ C, int M,
                       int N, int K, float alpha, float beta, int64_t strideA, int64_t strideB, int64_t strideC, int vec_a,
                       int vec_b, int vec_c, int splits, int k_chunk, float* __restrict__ partial) {
  // splits > 1 (split-K, for problems with too few tiles to fill the GPU): blockIdx.z = batch * splits + s, this CTA sums
  // k in [s * k_chunk, (s + 1) * k_chunk) and writes its raw fp32 sums to partial[s][batch][M][N]; splitk_reduce_kernel adds
  // the slices in increasing s and applies alpha / beta.
  static_assert(LBM == 128 || LBM == 64, "row tiles of 128 or 64");
  constexpr int RG = LBM / 64;       // groups of 4 rows per thread
  constexpr int TR = 4 * RG;         // rows per thread
  constexpr int EA = LBM * LBK / 1024;  // float4 slots of the A tile per thread
  __shared__ __align__(16) float As[2][LBK][LBM + 4];
  __shared__ __align__(16) float Bs[2][LBK][LBN + 4];
  const int batch = blockIdx.z / splits, split = blockIdx.z % splits;
  const int k_begin = split * k_chunk, k_end = min(K, k_begin + k_chunk);
  A += batch * strideA;
  B += batch * strideB;
  C += batch * strideC;
  const int m0 = blockIdx.y * LBM, n0 = blockIdx.x * LBN;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const bool a_kmajor = !a_trans;  // A stored [M, K]
  const bool b_kmajor = b_trans;   // B stored [N, K]
  const bool rows_in = m0 + LBM <= M, cols_in = n0 + LBN <= N;

  float acc[TR][8];
#pragma unroll
  for (int i = 0; i < TR; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  // Slot e of a thread: f = tid + 256 e. k-major operand: row f / 4, k offset 4 (f % 4), four along k.
  // Operand stored [K, R] (R = tile rows): k = f / (R / 4), rows 4 (f % (R / 4)) .. +3.
  float4 ra[EA], rb[2];
  auto fetch = [&](int k0) {
    const bool k_in = k0 + LBK <= k_end;
#pragma unroll
    for (int e = 0; e < EA; ++e) {
      const int f = tid + e * 256;
      if (a_kmajor) ra[e] = fetch4(A, vec_a, rows_in && k_in, m0 + f / 4, k0 + 4 * (f % 4), M, K, k_end, true);
      else ra[e] = fetch4(A, vec_a, rows_in && k_in, m0 + 4 * (f % (LBM / 4)), k0 + f / (LBM / 4), M, K, k_end, false);
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int f = tid + e * 256;
      if (b_kmajor) rb[e] = fetch4(B, vec_b, cols_in && k_in, n0 + f / 4, k0 + 4 * (f % 4), N, K, k_end, true);
      else rb[e] = fetch4(B, vec_b, cols_in && k_in, n0 + 4 * (f % 32), k0 + f / 32, N, K, k_end, false);
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int e = 0; e < EA; ++e) {
      const int f = tid + e * 256;
      if (a_kmajor) {
        const int r = f / 4, k = 4 * (f % 4);
        As[buf][k][r] = ra[e].x; As[buf][k + 1][r] = ra[e].y; As[buf][k + 2][r] = ra[e].z; As[buf][k + 3][r] = ra[e].w;
      } else {
        *reinterpret_cast<float4*>(&As[buf][f / (LBM / 4)][4 * (f % (LBM / 4))]) = ra[e];
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int f = tid + e * 256;
      if (b_kmajor) {
        const int r = f / 4, k = 4 * (f % 4);
        Bs[buf][k][r] = rb[e].x; Bs[buf][k + 1][r] = rb[e].y; Bs[buf][k + 2][r] = rb[e].z; Bs[buf][k + 3][r] = rb[e].w;
      } else {
        *reinterpret_cast<float4*>(&Bs[buf][f / 32][4 * (f % 32)]) = rb[e];
      }
    }
  };

  if (k_begin < k_end) {
    fetch(k_begin);
    stage(0);
  }
  __syncthreads();
  int buf = 0;
  for (int k0 = k_begin; k0 < k_end; k0 += LBK) {
    const bool more = k0 + LBK < k_end;
    if (more) fetch(k0 + LBK);
#pragma unroll
    for (int k = 0; k < LBK; ++k) {
      float a[TR];
#pragma unroll
      for (int g = 0; g < RG; ++g) {
        const float4 v = *reinterpret_cast<const float4*>(&As[buf][k][g * 64 + ty * 4]);
        a[4 * g] = v.x; a[4 * g + 1] = v.y; a[4 * g + 2] = v.z; a[4 * g + 3] = v.w;
      }
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < TR; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) stage(buf ^ 1);  // the other buffer was last read before the previous barrier
    __syncthreads();
    buf ^= 1;
  }

#pragma unroll
  for (int i = 0; i < TR; ++i) {
    const int gm = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
    if (gm >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gn = n0 + h * 64 + tx * 4;
      if (partial) {
        float* p = partial + (((int64_t)split * (gridDim.z / splits) + batch) * M + gm) * N + gn;
        if (N % 4 == 0 && gn + 3 < N) {
          *reinterpret_cast<float4*>(p) = make_float4(acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (gn + c < N) p[c] = acc[i][h * 4 + c];
        }
        continue;
      }
      T* dst = C + (int64_t)gm * N + gn;
      if constexpr (std::is_same<T, float>::value) {
        if (vec_c && gn + 3 < N) {
          float4 r = make_float4(alpha * acc[i][h * 4], alpha * acc[i][h * 4 + 1], alpha * acc[i][h * 4 + 2], alpha * acc[i][h * 4 + 3]);
          if (beta != 0.f) {
            const float4 old = *reinterpret_cast<const float4*>(dst);
            r.x += beta * old.x; r.y += beta * old.y; r.z += beta * old.z; r.w += beta * old.w;
          }
          *reinterpret_cast<float4*>(dst) = r;
          continue;
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (gn + c >= N) continue;
        float r = alpha * acc[i][h * 4 + c];
        if (beta != 0.f) r += beta * to_f(dst[c]);
        dst[c] = from_f<T>(r);
      }
    }
  }
}

// C = alpha * (partial[0] + partial[1] + ... in this order) + beta * C over `total` contiguous elements.
template <typename T>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t total, float alpha, float beta, T* __restrict__ C) {
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= total) return;
  float s = 0.f;
  for (int sp = 0; sp < splits; ++sp) s += partial[(int64_t)sp * total + idx];
  float r = alpha * s;
  if (beta != 0.f) r += beta * to_f(C[idx]);
  C[idx] = from_f<T>(r);
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
  // 128 x 128 tiles from two waves of them (two CTAs per SM); 64 x 128 from most of one wave; 64 x 64 below that
  const int64_t n128 = (N + 127) / 128;
  const bool wide = n128 * 128 * 4 <= N * 5;  // 128-column tiles carry at most a quarter of padding
  const bool large = wide && ((M + 127) / 128) * n128 * batch >= 4ll * ctx->sm_count;
  const bool medium = wide && !large && ((M + 63) / 64) * n128 * batch >= (3ll * ctx->sm_count) / 2;
  // Too few tiles and a long k: split k over CTAs (64 x 128 tiles, k slices of at least 64) and add the slices in a
  // second pass. Deterministic, but the sum is no longer in plain increasing-k order.
  int splits = 1, k_chunk = (int)K;
  if (small && wide && K >= 256) {
    const int64_t tiles = ((M + 63) / 64) * n128 * batch;
    int64_t want = std::min<int64_t>((2ll * ctx->sm_count + tiles - 1) / tiles, K / 64);
    if (want > 1 && want * batch <= 65535) {
      k_chunk = (int)(((K + want - 1) / want + 15) / 16 * 16);
      splits = (int)((K + k_chunk - 1) / k_chunk);
    }
  }
  if (splits > 1) {
    auto al16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    const bool f32 = dtype == TTB_F32;
    const int vec_a = f32 && al16(A) && (a_trans ? M % 4 == 0 : K % 4 == 0) && (M * K) % 4 == 0;
    const int vec_b = f32 && al16(B) && (b_trans ? K % 4 == 0 : N % 4 == 0) && (K * N) % 4 == 0;
    const int64_t total = batch * M * N;
    void* ws = nullptr;
    int s = ttb_alloc(ctx, (size_t)(splits * total) * sizeof(float), "matmul/split_k", &ws);
    if (s) return s;
    dim3 grid((unsigned)n128, (unsigned)((M + 63) / 64), (unsigned)(batch * splits));
    TTB_DISPATCH_FLOAT(ctx, dtype, T,
                       (gemm_simt_large_kernel<T, 64><<<grid, 256, 0, ctx->stream>>>((const T*)A, a_trans, (const T*)B, b_trans, (T*)C, (int)M, (int)N,
                                                                                    (int)K, alpha, beta, M * K, K * N, M * N, vec_a, vec_b, 0, splits,
                                                                                    k_chunk, (float*)ws)));
    s = launched(ctx, what);
    if (!s) {
      TTB_DISPATCH_FLOAT(ctx, dtype, T,
                         (splitk_reduce_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>((const float*)ws, splits, total, alpha, beta,
                                                                                                           (T*)C)));
      s = launched(ctx, what);
    }
    const int f = ttb_free(ctx, ws, "matmul/split_k");  // stream-ordered: released after the reduce has run
    return s ? s : f;
  }
  const int bm = small ? 32 : (large ? 128 : 64), bn = small ? 32 : ((large || medium) ? 128 : 64);
  const int64_t gy = (M + bm - 1) / bm, gx = (N + bn - 1) / bn;
  TTB_REQUIRE(ctx, gy <= 65535, "%s: M too large for this kernel", what);
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (int)(batch - b0 < 65535 ? batch - b0 : 65535);
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)nb);
    if (small) {
      TTB_DISPATCH_FLOAT(ctx, dtype, T,
                         (gemm_simt_kernel<T, 32, 32, 2, 2, 64><<<grid, 256, 0, ctx->stream>>>((const T*)A + b0 * M * K, a_trans, (const T*)B + b0 * K * N,
                                                                                          b_trans, (T*)C + b0 * M * N, (int)M, (int)N, (int)K,
                                                                                          alpha, beta, M * K, K * N, M * N)));
    } else if (large || medium) {
      // float4 access: fp32, 16-byte aligned bases, and every row (and every batch member) starting on a 16-byte boundary
      auto al16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
      const bool f32 = dtype == TTB_F32;
      const int vec_a = f32 && al16(A) && (a_trans ? M % 4 == 0 : K % 4 == 0) && (M * K) % 4 == 0;
      const int vec_b = f32 && al16(B) && (b_trans ? K % 4 == 0 : N % 4 == 0) && (K * N) % 4 == 0;
      const int vec_c = f32 && al16(C) && N % 4 == 0;
      if (large) {
        TTB_DISPATCH_FLOAT(ctx, dtype, T,
                           (gemm_simt_large_kernel<T, 128><<<grid, 256, 0, ctx->stream>>>((const T*)A + b0 * M * K, a_trans, (const T*)B + b0 * K * N,
                                                                                         b_trans, (T*)C + b0 * M * N, (int)M, (int)N, (int)K, alpha,
                                                                                         beta, M * K, K * N, M * N, vec_a, vec_b, vec_c, 1, (int)K, nullptr)));
      } else {
        TTB_DISPATCH_FLOAT(ctx, dtype, T,
                           (gemm_simt_large_kernel<T, 64><<<grid, 256, 0, ctx->stream>>>((const T*)A + b0 * M * K, a_trans, (const T*)B + b0 * K * N,
                                                                                        b_trans, (T*)C + b0 * M * N, (int)M, (int)N, (int)K, alpha,
                                                                                        beta, M * K, K * N, M * N, vec_a, vec_b, vec_c, 1, (int)K, nullptr)));
      }
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
