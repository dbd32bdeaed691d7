// Bandwidth-bound kernels: layer norm, bias/activation, embedding, pooling, transposes, softmax, quantise.
// All are warp-per-row or 16-byte-vector grid-stride kernels; reductions use warp shuffles and fp32 math.
#include <type_traits>
#include <vector>

#include "ttb_common.cuh"
#include "ttb_sm100.cuh"

using namespace ttb;

namespace {

constexpr int kRowsPerBlock = 4;  // warps per CTA in warp-per-row kernels

inline int grid_for(int64_t work, int per_block, int sm_count) {
  int64_t g = (work + per_block - 1) / per_block;
  int64_t cap = (int64_t)sm_count * 32;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// ------------------------------------------------------------------------------------------------
// LayerNorm: out = LN(x [+ residual + bias]) * gamma + beta. One warp per pair of rows, both rows cached in registers
// and all of their loads issued before the first reduction, so that a warp keeps 2 x N elements in flight.
// ITERS vectors of 8 elements per lane and row: N % 8 == 0 and N <= 256*ITERS. x may be out (no __restrict__ on them).
// TIn is the type of x / residual, TOut of gamma / beta / bias / out. EXTRA adds two optional outputs for models that
// carry more precision than TOut between layers: out_lo = what rounding to TOut dropped, out_f32 = the fp32 value.
// ------------------------------------------------------------------------------------------------
constexpr int kLnWarps = 8;
constexpr int kLnRows = 2;

template <typename TIn, typename TOut, int ITERS, bool ADD, bool EXTRA>
__global__ void __launch_bounds__(kLnWarps * 32)
layernorm_rows_kernel(const TIn* x, const TIn* __restrict__ residual, const TOut* __restrict__ bias, const TOut* __restrict__ gamma,
                      const TOut* __restrict__ beta, TOut* out, TOut* __restrict__ out_lo, float* __restrict__ out_f32, int64_t M, int N,
                      float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * kLnWarps;
  for (int64_t row0 = ((int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5)) * kLnRows; row0 < M; row0 += warps_total * kLnRows) {
    float v[kLnRows][ITERS][8];
    float sum[kLnRows];
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) {
      sum[r] = 0.f;
      const int64_t row = row0 + r;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        if (row < M && col < N) {
          Vec8<TIn> a;
          a.load(x + row * N + col);
          if (ADD) {
            Vec8<TIn> rs;
            Vec8<TOut> b;
            rs.load(residual + row * N + col);
            b.load(bias + col);
#pragma unroll
            for (int j = 0; j < 8; ++j) a.v[j] = a.v[j] + rs.v[j] + b.v[j];
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) { v[r][it][j] = a.v[j]; sum[r] += a.v[j]; }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[r][it][j] = 0.f;
        }
      }
    }
    float mean[kLnRows], sq[kLnRows];
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) mean[r] = warp_sum(sum[r]) / (float)N;
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) {
      sq[r] = 0.f;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        if (col < N) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { float d = v[r][it][j] - mean[r]; sq[r] += d * d; }
        }
      }
    }
    float rstd[kLnRows];
#pragma unroll
    for (int r = 0; r < kLnRows; ++r) rstd[r] = rsqrtf(warp_sum(sq[r]) / (float)N + eps);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int col = (it * 32 + lane) * 8;
      if (col < N) {
        Vec8<TOut> g, b;
        g.load(gamma + col);
        b.load(beta + col);
#pragma unroll
        for (int r = 0; r < kLnRows; ++r) {
          const int64_t row = row0 + r;
          if (row < M) {
            Vec8<TOut> o;
#pragma unroll
            for (int j = 0; j < 8; ++j) o.v[j] = b.v[j] + g.v[j] * rstd[r] * (v[r][it][j] - mean[r]);
            o.store(out + row * N + col);
            if (EXTRA) {
              if (out_f32) {
                Vec8<float> f;
#pragma unroll
                for (int j = 0; j < 8; ++j) f.v[j] = o.v[j];
                f.store(out_f32 + row * N + col);
              }
              if (out_lo) {
                Vec8<TOut> l;
#pragma unroll
                for (int j = 0; j < 8; ++j) l.v[j] = o.v[j] - to_f(from_f<TOut>(o.v[j]));
                l.store(out_lo + row * N + col);
              }
            }
          }
        }
      }
    }
  }
}

// The same for 16-bit rows without the residual form (the 16-bit models' hot case), as a streaming kernel: a grid that
// just fills the machine, every warp walking batches of two rows and issuing the loads of its next batch before it
// works on the current one, so that loads, arithmetic and stores of different batches overlap inside every warp. The
// rows stay in registers as they were loaded (packed 16-bit); gamma and beta sit in shared memory as fp32, converted
// once per CTA. About 190 instructions per row at N = 768 (the one-batch-per-warp form it replaces: 340, with all the
// warps of a wave loading at the same time and then computing at the same time).
constexpr int kLn16Rows = 2;
constexpr int kLn16MaxN = 1024;

// The row arithmetic the 16-bit LayerNorm kernels share (so that they agree bit for bit): both moments in one pass,
// var = E[x^2] - mean^2 as the reference's CPU kernel computes it (layer_norm.cpp:58-66), and the value as two fused
// multiply-adds, ((x * rstd) - mean * rstd) * gamma + beta.
__device__ __forceinline__ void ln_row_params(float sum, float sq, float inv_n, float eps, float& rstd, float& shift) {
  const float mean = sum * inv_n;
  const float var = fmaxf(sq * inv_n - mean * mean, 0.f);
  rstd = rsqrtf(var + eps);
  shift = -mean * rstd;
}
__device__ __forceinline__ float ln_value(float x, float rstd, float shift, float g, float b) { return fmaf(fmaf(x, rstd, shift), g, b); }

template <typename T, int ITERS, bool EXTRA>
__global__ void __launch_bounds__(kLnWarps * 32, 2)
layernorm16_stream_kernel(const T* x, const T* __restrict__ gamma, const T* __restrict__ beta, T* out, T* __restrict__ out_lo,
                          float* __restrict__ out_f32, int64_t M, int N, float eps) {
  __shared__ __align__(16) float s_gamma[ITERS * 256], s_beta[ITERS * 256];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t stride = (int64_t)gridDim.x * kLnWarps;
  const int64_t batches = (M + kLn16Rows - 1) / kLn16Rows;
  const float inv_n = 1.0f / (float)N;

  auto load = [&](uint4 (&raw)[kLn16Rows][ITERS], int64_t batch) {
#pragma unroll
    for (int r = 0; r < kLn16Rows; ++r) {
      const int64_t row = batch * kLn16Rows + r;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        raw[r][it] = (row < M && col < N) ? *reinterpret_cast<const uint4*>(x + row * N + col) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto unpack = [](const uint4& q, float (&f)[8]) {
    const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = to_f(h[j]);
  };
  auto work = [&](uint4 (&raw)[kLn16Rows][ITERS], int64_t batch) {
    // one pass for both moments, var = E[x^2] - mean^2 as the reference's CPU kernel computes it (layer_norm.cpp:58-66)
    float sum[kLn16Rows], sq[kLn16Rows];
#pragma unroll
    for (int r = 0; r < kLn16Rows; ++r) {
      sum[r] = 0.f;
      sq[r] = 0.f;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        float f[8];
        unpack(raw[r][it], f);  // lanes beyond N hold zeros
#pragma unroll
        for (int j = 0; j < 8; ++j) { sum[r] += f[j]; sq[r] = fmaf(f[j], f[j], sq[r]); }
        // the packed words stay the only live copy of the row: the second pass converts them again
        asm volatile("" : "+r"(raw[r][it].x), "+r"(raw[r][it].y), "+r"(raw[r][it].z), "+r"(raw[r][it].w));
      }
    }
    float rstd[kLn16Rows], shift[kLn16Rows];  // (x - mean) * rstd = x * rstd + shift
#pragma unroll
    for (int r = 0; r < kLn16Rows; ++r) ln_row_params(warp_sum(sum[r]), warp_sum(sq[r]), inv_n, eps, rstd[r], shift[r]);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int col = (it * 32 + lane) * 8;
      if (col < N) {
        float g[8], b[8];
        *reinterpret_cast<float4*>(&g[0]) = *reinterpret_cast<const float4*>(&s_gamma[col]);
        *reinterpret_cast<float4*>(&g[4]) = *reinterpret_cast<const float4*>(&s_gamma[col + 4]);
        *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(&s_beta[col]);
        *reinterpret_cast<float4*>(&b[4]) = *reinterpret_cast<const float4*>(&s_beta[col + 4]);
#pragma unroll
        for (int r = 0; r < kLn16Rows; ++r) {
          const int64_t row = batch * kLn16Rows + r;
          if (row < M) {
            float f[8];
            unpack(raw[r][it], f);
            Vec8<T> o;
#pragma unroll
            for (int j = 0; j < 8; ++j) o.v[j] = ln_value(f[j], rstd[r], shift[r], g[j], b[j]);
            o.store(out + row * N + col);
            if (EXTRA) {
              if (out_f32) {
                Vec8<float> w;
#pragma unroll
                for (int j = 0; j < 8; ++j) w.v[j] = o.v[j];
                w.store(out_f32 + row * N + col);
              }
              if (out_lo) {
                Vec8<T> l;
#pragma unroll
                for (int j = 0; j < 8; ++j) l.v[j] = o.v[j] - to_f(from_f<T>(o.v[j]));
                l.store(out_lo + row * N + col);
              }
            }
          }
        }
      }
    }
  };

  uint4 a[kLn16Rows][ITERS], b[kLn16Rows][ITERS];
  int64_t batch = (int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  if (batch < batches) load(a, batch);
  for (int c = threadIdx.x; c < ITERS * 256; c += kLnWarps * 32) {  // in the shadow of the first rows' loads
    s_gamma[c] = c < N ? to_f(gamma[c]) : 0.f;
    s_beta[c] = c < N ? to_f(beta[c]) : 0.f;
  }
  __syncthreads();
  while (batch < batches) {
    if (batch + stride < batches) load(b, batch + stride);
    work(a, batch);
    batch += stride;
    if (batch >= batches) break;
    if (batch + stride < batches) load(a, batch + stride);
    work(b, batch);
    batch += stride;
  }
}

// Few rows (a single short request): one row per warp, the row and its gamma / beta slices all requested before the first
// use, no shared memory and no block barrier: the kernel is one memory round trip long.
template <typename T, int ITERS, bool EXTRA>
__global__ void __launch_bounds__(kLnWarps * 32)
layernorm16_small_kernel(const T* x, const T* __restrict__ gamma, const T* __restrict__ beta, T* out, T* __restrict__ out_lo,
                         float* __restrict__ out_f32, int64_t M, int N, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  if (row >= M) return;
  uint4 raw[ITERS], gq[ITERS], bq[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int col = (it * 32 + lane) * 8;
    const bool in = col < N;
    raw[it] = in ? *reinterpret_cast<const uint4*>(x + row * N + col) : make_uint4(0, 0, 0, 0);
    gq[it] = in ? *reinterpret_cast<const uint4*>(gamma + col) : make_uint4(0, 0, 0, 0);
    bq[it] = in ? *reinterpret_cast<const uint4*>(beta + col) : make_uint4(0, 0, 0, 0);
  }
  float sum = 0.f, sq = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const T* h = reinterpret_cast<const T*>(&raw[it]);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float f = to_f(h[j]); sum += f; sq = fmaf(f, f, sq); }
  }
  float rstd, shift;
  ln_row_params(warp_sum(sum), warp_sum(sq), 1.0f / (float)N, eps, rstd, shift);
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int col = (it * 32 + lane) * 8;
    if (col < N) {
      const T* h = reinterpret_cast<const T*>(&raw[it]);
      const T* g = reinterpret_cast<const T*>(&gq[it]);
      const T* b = reinterpret_cast<const T*>(&bq[it]);
      Vec8<T> o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] = ln_value(to_f(h[j]), rstd, shift, to_f(g[j]), to_f(b[j]));
      o.store(out + row * N + col);
      if (EXTRA) {
        if (out_f32) {
          Vec8<float> w;
#pragma unroll
          for (int j = 0; j < 8; ++j) w.v[j] = o.v[j];
          w.store(out_f32 + row * N + col);
        }
        if (out_lo) {
          Vec8<T> l;
#pragma unroll
          for (int j = 0; j < 8; ++j) l.v[j] = o.v[j] - to_f(from_f<T>(o.v[j]));
          l.store(out_lo + row * N + col);
        }
      }
    }
  }
}

// Large row counts: the same arithmetic fed by bulk copies. One CTA per SM; a producer thread streams chunks of 32 rows
// (contiguous in memory) into a ring of shared-memory stages with cp.async.bulk, 16 consumer warps take two rows of a
// chunk each into registers, release the stage and normalise. The depth of the prefetch is the ring (up to 192 KB per SM
// in flight), not the register file, and every wait is bounded.
constexpr int kLnTmaConsumers = 8;
constexpr int kLnTmaRows = 16;
constexpr int kLnTmaMaxStages = 6;
constexpr int kLnTmaCtasPerSm = 2;
constexpr size_t kLnTmaSmem = 100 * 1024;

template <typename T, int ITERS, bool EXTRA>
__global__ void __launch_bounds__((kLnTmaConsumers + 1) * 32, kLnTmaCtasPerSm)
layernorm16_tma_kernel(const T* x, const T* __restrict__ gamma, const T* __restrict__ beta, T* out, T* __restrict__ out_lo,
                       float* __restrict__ out_f32, int64_t M, int N, float eps, int stages, int* status) {
  using namespace ttb::sm100;
  extern __shared__ __align__(128) uint8_t ln_smem[];
  const uint32_t stage_bytes = (uint32_t)(kLnTmaRows * N * (int)sizeof(T));
  float* s_gamma = reinterpret_cast<float*>(ln_smem + (size_t)stages * stage_bytes);
  float* s_beta = s_gamma + N;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_beta + N);  // full[stages], empty[stages]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kLnTmaMaxStages);
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int st) { return bar0 + 8u * (uint32_t)st; };
  auto empty = [&](int st) { return bar0 + 8u * (uint32_t)(kLnTmaMaxStages + st); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int st = 0; st < stages; ++st) {
      mbar_init(full(st), 1);
      mbar_init(empty(st), kLnTmaConsumers);
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  pdl_trigger();
  __syncthreads();  // barriers initialised
  pdl_wait();
  const int64_t chunks = (M + kLnTmaRows - 1) / kLnTmaRows;
  if (warp != kLnTmaConsumers) {  // gamma / beta, in the shadow of the first chunks' copies (the producer does not wait for them)
    for (int c = threadIdx.x; c < N; c += kLnTmaConsumers * 32) {
      s_gamma[c] = to_f(gamma[c]);
      s_beta[c] = to_f(beta[c]);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kLnTmaConsumers * 32) : "memory");
  }
  if (warp == kLnTmaConsumers) {
    if (lane == 0) {
      uint32_t n = 0;
      for (int64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x, ++n) {
        const int st = (int)(n % (uint32_t)stages);
        const uint32_t round = n / (uint32_t)stages;
        if (!mbar_wait(empty(st), (round & 1u) ^ 1u, abort_flag)) break;
        const int64_t rows = min((int64_t)kLnTmaRows, M - chunk * kLnTmaRows);
        const uint32_t bytes = (uint32_t)(rows * N * (int64_t)sizeof(T));  // a multiple of 16: N is a multiple of 8
        mbar_expect_tx(full(st), bytes);
        bulk_load_1d(smem_u32(ln_smem) + (uint32_t)st * stage_bytes, x + chunk * kLnTmaRows * N, bytes, full(st));
      }
      if (*abort_flag) {  // let copies in flight land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) {
        }
      }
    }
    __syncwarp();
  } else {
    const float inv_n = 1.0f / (float)N;
    uint32_t n = 0;
    for (int64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x, ++n) {
      const int st = (int)(n % (uint32_t)stages);
      const uint32_t round = n / (uint32_t)stages;
      if (!__all_sync(0xffffffffu, mbar_wait(full(st), round & 1u, abort_flag))) break;
      const T* src = reinterpret_cast<const T*>(ln_smem + (size_t)st * stage_bytes);
      const int64_t row_base = chunk * kLnTmaRows;
      uint4 raw[2][ITERS];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int lr = warp + r * kLnTmaConsumers;  // row within the chunk
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
          const int col = (it * 32 + lane) * 8;
          raw[r][it] = (row_base + lr < M && col < N) ? *reinterpret_cast<const uint4*>(src + lr * N + col) : make_uint4(0, 0, 0, 0);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(st));  // the rows are in registers: the stage may be refilled
      float sum[2] = {0.f, 0.f}, sq[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 2; ++r) {
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
          const T* h = reinterpret_cast<const T*>(&raw[r][it]);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float f = to_f(h[j]); sum[r] += f; sq[r] = fmaf(f, f, sq[r]); }
          asm volatile("" : "+r"(raw[r][it].x), "+r"(raw[r][it].y), "+r"(raw[r][it].z), "+r"(raw[r][it].w));
        }
      }
      float rstd[2], shift[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) ln_row_params(warp_sum(sum[r]), warp_sum(sq[r]), inv_n, eps, rstd[r], shift[r]);
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        if (col < N) {
          float g[8], b[8];
          *reinterpret_cast<float4*>(&g[0]) = *reinterpret_cast<const float4*>(&s_gamma[col]);
          *reinterpret_cast<float4*>(&g[4]) = *reinterpret_cast<const float4*>(&s_gamma[col + 4]);
          *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(&s_beta[col]);
          *reinterpret_cast<float4*>(&b[4]) = *reinterpret_cast<const float4*>(&s_beta[col + 4]);
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int64_t row = row_base + warp + r * kLnTmaConsumers;
            if (row < M) {
              const T* h = reinterpret_cast<const T*>(&raw[r][it]);
              Vec8<T> o;
#pragma unroll
              for (int j = 0; j < 8; ++j) o.v[j] = ln_value(to_f(h[j]), rstd[r], shift[r], g[j], b[j]);
              o.store(out + row * N + col);
              if (EXTRA) {
                if (out_f32) {
                  Vec8<float> w;
#pragma unroll
                  for (int j = 0; j < 8; ++j) w.v[j] = o.v[j];
                  w.store(out_f32 + row * N + col);
                }
                if (out_lo) {
                  Vec8<T> l;
#pragma unroll
                  for (int j = 0; j < 8; ++j) l.v[j] = o.v[j] - to_f(from_f<T>(o.v[j]));
                  l.store(out_lo + row * N + col);
                }
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(status, (int)TTB_ERR_DEVICE_WAIT);
}

// Any N: one warp per row, three passes over the row (the re-reads hit L1/L2).
template <typename TIn, typename TOut, bool ADD>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
layernorm_rows_generic_kernel(const TIn* x, const TIn* __restrict__ residual, const TOut* __restrict__ bias, const TOut* __restrict__ gamma,
                              const TOut* __restrict__ beta, TOut* out, TOut* __restrict__ out_lo, float* __restrict__ out_f32, int64_t M,
                              int N, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * kRowsPerBlock;
  for (int64_t row = (int64_t)blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5); row < M; row += warps_total) {
    auto val = [&](int c) {
      float a = to_f(x[row * N + c]);
      if (ADD) a += to_f(residual[row * N + c]) + to_f(bias[c]);
      return a;
    };
    float sum = 0.f;
    for (int c = lane; c < N; c += 32) sum += val(c);
    const float mean = warp_sum(sum) / (float)N;
    float sq = 0.f;
    for (int c = lane; c < N; c += 32) { float d = val(c) - mean; sq += d * d; }
    const float rstd = rsqrtf(warp_sum(sq) / (float)N + eps);
    // x may alias out: every lane reads only the columns it then writes.
    for (int c = lane; c < N; c += 32) {
      const float y = to_f(beta[c]) + to_f(gamma[c]) * rstd * (val(c) - mean);
      out[row * N + c] = from_f<TOut>(y);
      if (out_f32) out_f32[row * N + c] = y;
      if (out_lo) out_lo[row * N + c] = from_f<TOut>(y - to_f(from_f<TOut>(y)));
    }
  }
}

template <typename TIn, typename TOut, bool ADD>
int launch_layernorm(ttb_ctx* ctx, const TIn* x, const TIn* residual, const TOut* bias, const TOut* gamma, const TOut* beta, TOut* out,
                     TOut* out_lo, float* out_f32, int64_t M, int64_t N, float eps) {
  if (M == 0) return TTB_OK;
  const int64_t pair_warps = (M + kLnRows - 1) / kLnRows;
  const int grid = grid_for(pair_warps, kLnWarps, ctx->sm_count);
  const int block = kLnWarps * 32;
  const bool extra = out_lo != nullptr || out_f32 != nullptr;
#define LN_CASE(IT)                                                                                                              \
  do {                                                                                                                           \
    if (extra)                                                                                                                   \
      launch_pdl(layernorm_rows_kernel<TIn, TOut, IT, ADD, true>, dim3(grid), dim3(block), 0, ctx->stream, x, residual, bias, gamma, beta, \
                 out, out_lo, out_f32, M, (int)N, eps);                                                                          \
    else                                                                                                                         \
      launch_pdl(layernorm_rows_kernel<TIn, TOut, IT, ADD, false>, dim3(grid), dim3(block), 0, ctx->stream, x, residual, bias, gamma, beta, \
                 out, out_lo, out_f32, M, (int)N, eps);                                                                          \
  } while (0)
  const bool aligned = (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out_lo) |
                                         reinterpret_cast<uintptr_t>(out_f32) | reinterpret_cast<uintptr_t>(gamma) |
                                         reinterpret_cast<uintptr_t>(beta) |
                                         (ADD ? (reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(bias)) : 0)) %
                                            16 == 0);
  if constexpr (!ADD && std::is_same<TIn, TOut>::value && sizeof(TIn) == 2) {
    const int64_t chunks = (M + kLnTmaRows - 1) / kLnTmaRows;
    static const bool tma_off = [] { const char* e = getenv("TTB_LN_TMA"); return e && e[0] == '0'; }();
    if (!tma_off && aligned && N <= kLn16MaxN && chunks >= 2 * (int64_t)ctx->sm_count && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
      const size_t stage_bytes = (size_t)kLnTmaRows * N * sizeof(TOut);
      const size_t fixed = (size_t)2 * N * sizeof(float) + 2 * kLnTmaMaxStages * 8 + 16;
      const int stages = (int)std::min<size_t>(kLnTmaMaxStages, (kLnTmaSmem - fixed) / stage_bytes);
      const size_t smem = (size_t)stages * stage_bytes + fixed;
      const int grid = (int)std::min<int64_t>(chunks, (int64_t)ctx->sm_count * kLnTmaCtasPerSm);
#define LNT_CASE(IT)                                                                                                                   \
  do {                                                                                                                                 \
    auto kern = extra ? layernorm16_tma_kernel<TOut, IT, true> : layernorm16_tma_kernel<TOut, IT, false>;                              \
    static bool configured[2][64] = {};                                                                                                \
    if (ctx->device < 64 && !configured[extra ? 1 : 0][ctx->device]) {                                                                 \
      TTB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLnTmaSmem));                            \
      configured[extra ? 1 : 0][ctx->device] = true;                                                                                   \
    }                                                                                                                                  \
    launch_pdl(kern, dim3(grid), dim3((kLnTmaConsumers + 1) * 32), smem, ctx->stream, x, gamma, beta, out, out_lo, out_f32, M, (int)N, \
               eps, stages, ctx->d_status);                                                                                            \
  } while (0)
      if (N <= 256) LNT_CASE(1);
      else if (N <= 512) LNT_CASE(2);
      else if (N <= 768) LNT_CASE(3);
      else LNT_CASE(4);
#undef LNT_CASE
      return launched(ctx, "layernorm");
    }
    if (aligned && N <= kLn16MaxN && M <= 8 * (int64_t)ctx->sm_count) {  // at most one CTA of single-row warps per SM
      const int grid1 = (int)((M + kLnWarps - 1) / kLnWarps);
#define LNS_CASE(IT)                                                                                                                   \
  do {                                                                                                                                 \
    if (extra)                                                                                                                         \
      launch_pdl(layernorm16_small_kernel<TOut, IT, true>, dim3(grid1), dim3(block), 0, ctx->stream, x, gamma, beta, out, out_lo, out_f32, M, \
                 (int)N, eps);                                                                                                         \
    else                                                                                                                               \
      launch_pdl(layernorm16_small_kernel<TOut, IT, false>, dim3(grid1), dim3(block), 0, ctx->stream, x, gamma, beta, out, out_lo, out_f32, M, \
                 (int)N, eps);                                                                                                         \
  } while (0)
      if (N <= 256) LNS_CASE(1);
      else if (N <= 512) LNS_CASE(2);
      else if (N <= 768) LNS_CASE(3);
      else LNS_CASE(4);
#undef LNS_CASE
      return launched(ctx, "layernorm");
    }
    if (aligned && N <= kLn16MaxN) {
      // two CTAs per SM are resident; fewer CTAs when the rows do not fill them
      const int64_t batches = (M + kLn16Rows - 1) / kLn16Rows;
      const int grid16 = (int)std::min<int64_t>((batches + kLnWarps - 1) / kLnWarps, (int64_t)ctx->sm_count * 2);
#define LN16_CASE(IT)                                                                                                                  \
  do {                                                                                                                                 \
    if (extra)                                                                                                                         \
      launch_pdl(layernorm16_stream_kernel<TOut, IT, true>, dim3(grid16), dim3(block), 0, ctx->stream, x, gamma, beta, out, out_lo, out_f32, M, \
                 (int)N, eps);                                                                                                         \
    else                                                                                                                               \
      launch_pdl(layernorm16_stream_kernel<TOut, IT, false>, dim3(grid16), dim3(block), 0, ctx->stream, x, gamma, beta, out, out_lo, out_f32, M, \
                 (int)N, eps);                                                                                                         \
  } while (0)
      if (N <= 256) LN16_CASE(1);
      else if (N <= 512) LN16_CASE(2);
      else if (N <= 768) LN16_CASE(3);
      else LN16_CASE(4);
#undef LN16_CASE
      return launched(ctx, "layernorm");
    }
  }
  if (aligned && N <= 256) LN_CASE(1);
  else if (aligned && N <= 512) LN_CASE(2);
  else if (aligned && N <= 768) LN_CASE(3);
  else if (aligned && N <= 1024) LN_CASE(4);
  else if (aligned && N <= 2048) LN_CASE(8);
  else
    layernorm_rows_generic_kernel<TIn, TOut, ADD><<<grid_for(M, kRowsPerBlock, ctx->sm_count), kRowsPerBlock * 32, 0, ctx->stream>>>(
        x, residual, bias, gamma, beta, out, out_lo, out_f32, M, (int)N, eps);
#undef LN_CASE
  return launched(ctx, "layernorm");
}

// ------------------------------------------------------------------------------------------------
// out = act(out + bias), in place.
// ------------------------------------------------------------------------------------------------
template <int ACT> __device__ __forceinline__ float apply_act(float x) {
  if (ACT == TTB_ACT_GELU) return gelu_tanh(x);
  if (ACT == TTB_ACT_TANH) return tanhf(x);
  return x > 0.f ? x : 0.f;
}

template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(256)
add_bias_act_kernel(T* __restrict__ out, const T* __restrict__ bias, int64_t M, int N) {
  if (VEC) {
    const int64_t nvec = M * (int64_t)(N / 8);
    const int per_row = N / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
      const int col = (int)(i % per_row) * 8;
      Vec8<T> a, b;
      a.load(out + i * 8);
      b.load(bias + col);
#pragma unroll
      for (int j = 0; j < 8; ++j) a.v[j] = apply_act<ACT>(a.v[j] + b.v[j]);
      a.store(out + i * 8);
    }
  } else {
    const int64_t n = M * (int64_t)N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
      out[i] = from_f<T>(apply_act<ACT>(to_f(out[i]) + to_f(bias[i % N])));
  }
}

// out = in1 (+ in2) + bias
template <typename T, bool ADD_INPUT>
__global__ void __launch_bounds__(256)
add_bias_kernel(const T* __restrict__ in1, const T* __restrict__ in2, const T* __restrict__ bias, T* __restrict__ out,
                int64_t M, int N) {
  const int64_t n = M * (int64_t)N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float a = to_f(in1[i]) + to_f(bias[i % N]);
    if (ADD_INPUT) a += to_f(in2[i]);
    out[i] = from_f<T>(a);
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding gather. Ids outside the table are clamped and flagged (the reference trapped the GPU).
// ------------------------------------------------------------------------------------------------
template <typename T, bool ADD>
__global__ void __launch_bounds__(256)
lookup_kernel(T* __restrict__ out, const T* __restrict__ table, const int64_t* __restrict__ ids, int64_t n_ids,
              int hidden, int64_t vocab, int* status) {
  for (int64_t r = blockIdx.x; r < n_ids; r += gridDim.x) {
    int64_t id = ids[r];
    if (id < 0 || id >= vocab) {
      if (threadIdx.x == 0) atomicExch(status, (int)TTB_ERR_BAD_INDEX);
      id = id < 0 ? 0 : vocab - 1;
    }
    const T* src = table + id * hidden;
    T* dst = out + r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
      dst[c] = ADD ? from_f<T>(to_f(dst[c]) + to_f(src[c])) : src[c];
  }
}

__device__ __forceinline__ int find_sequence(const int32_t* cu, int B, int token) {
  int lo = 0, hi = B;  // largest b with cu[b] <= token
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu[mid] <= token) lo = mid; else hi = mid;
  }
  return lo;
}

// word[id] + position[pos] + token_type[tt] -> LayerNorm, one warp per token, any hidden size.
template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
embedding_ln_kernel(const int64_t* __restrict__ ids, const int64_t* __restrict__ pos_ids,
                    const int64_t* __restrict__ type_ids, const int32_t* __restrict__ cu, int B, int seq_len,
                    int64_t n_tokens, const T* __restrict__ word, const T* __restrict__ position,
                    const T* __restrict__ token_type, const T* __restrict__ gamma, const T* __restrict__ beta,
                    int hidden, int64_t vocab, int64_t n_pos, int64_t n_types, float eps, T* __restrict__ out,
                    T* __restrict__ out_lo, float* __restrict__ out_f32, int* status) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * kRowsPerBlock;
  for (int64_t t = (int64_t)blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5); t < n_tokens; t += warps_total) {
    int64_t id = ids[t];
    int64_t pos = pos_ids ? pos_ids[t] : (cu ? (int64_t)t - cu[find_sequence(cu, B, (int)t)] : (t % seq_len));
    int64_t tt = type_ids ? type_ids[t] : 0;
    bool bad = id < 0 || id >= vocab || pos < 0 || pos >= n_pos || tt < 0 || tt >= n_types;
    if (bad) {
      if (lane == 0) atomicExch(status, (int)TTB_ERR_BAD_INDEX);
      id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
      pos = pos < 0 ? 0 : (pos >= n_pos ? n_pos - 1 : pos);
      tt = tt < 0 ? 0 : (tt >= n_types ? n_types - 1 : tt);
    }
    const T* w = word + id * hidden;
    const T* p = position + pos * hidden;
    const T* y = token_type + tt * hidden;
    // same accumulation order as the reference: word, then token type, then position
    auto val = [&](int c) { return (to_f(w[c]) + to_f(y[c])) + to_f(p[c]); };
    float sum = 0.f;
    for (int c = lane; c < hidden; c += 32) sum += val(c);
    const float mean = warp_sum(sum) / (float)hidden;
    float sq = 0.f;
    for (int c = lane; c < hidden; c += 32) { float d = val(c) - mean; sq += d * d; }
    const float rstd = rsqrtf(warp_sum(sq) / (float)hidden + eps);
    for (int c = lane; c < hidden; c += 32) {
      const float y = to_f(beta[c]) + to_f(gamma[c]) * rstd * (val(c) - mean);
      out[t * hidden + c] = from_f<T>(y);
      if (out_f32) out_f32[t * hidden + c] = y;
      if (out_lo) out_lo[t * hidden + c] = from_f<T>(y - to_f(from_f<T>(y)));
    }
  }
}

// The same for 16-bit tables with hidden % 8 == 0 and hidden <= 256 * ITERS: 16-byte loads of the three rows, the sum held
// in registers for the two passes of the statistics and the output.
template <typename T, int ITERS>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
embedding_ln16_kernel(const int64_t* __restrict__ ids, const int64_t* __restrict__ pos_ids, const int64_t* __restrict__ type_ids,
                      const int32_t* __restrict__ cu, int B, int seq_len, int64_t n_tokens, const T* __restrict__ word,
                      const T* __restrict__ position, const T* __restrict__ token_type, const T* __restrict__ gamma,
                      const T* __restrict__ beta, int hidden, int64_t vocab, int64_t n_pos, int64_t n_types, float eps, T* __restrict__ out,
                      T* __restrict__ out_lo, float* __restrict__ out_f32, int* status) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * kRowsPerBlock;
  for (int64_t t = (int64_t)blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5); t < n_tokens; t += warps_total) {
    int64_t id = ids[t];
    int64_t pos = pos_ids ? pos_ids[t] : (cu ? (int64_t)t - cu[find_sequence(cu, B, (int)t)] : (t % seq_len));
    int64_t tt = type_ids ? type_ids[t] : 0;
    const bool bad = id < 0 || id >= vocab || pos < 0 || pos >= n_pos || tt < 0 || tt >= n_types;
    if (bad) {
      if (lane == 0) atomicExch(status, (int)TTB_ERR_BAD_INDEX);
      id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
      pos = pos < 0 ? 0 : (pos >= n_pos ? n_pos - 1 : pos);
      tt = tt < 0 ? 0 : (tt >= n_types ? n_types - 1 : tt);
    }
    const T* w = word + id * hidden;
    const T* p = position + pos * hidden;
    const T* y = token_type + tt * hidden;
    float v[ITERS][8];
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int col = (it * 32 + lane) * 8;
      if (col < hidden) {
        Vec8<T> a, b, c;
        a.load(w + col);
        b.load(y + col);
        c.load(p + col);
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // same accumulation order as the reference: word, then token type, then position
          v[it][j] = (a.v[j] + b.v[j]) + c.v[j];
          sum += v[it][j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[it][j] = 0.f;
      }
    }
    const float mean = warp_sum(sum) / (float)hidden;
    float sq = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      if ((it * 32 + lane) * 8 < hidden) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[it][j] - mean; sq += d * d; }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int col = (it * 32 + lane) * 8;
      if (col < hidden) {
        Vec8<T> g, b, o;
        g.load(gamma + col);
        b.load(beta + col);
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = b.v[j] + g.v[j] * rstd * (v[it][j] - mean);
        o.store(out + t * hidden + col);
        if (out_f32) {
          Vec8<float> f;
#pragma unroll
          for (int j = 0; j < 8; ++j) f.v[j] = o.v[j];
          f.store(out_f32 + t * hidden + col);
        }
        if (out_lo) {
          Vec8<T> l;
#pragma unroll
          for (int j = 0; j < 8; ++j) l.v[j] = o.v[j] - to_f(from_f<T>(o.v[j]));
          l.store(out_lo + t * hidden + col);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Pooling over the sequence axis.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void seq_pool_kernel(const T* __restrict__ in, int64_t B, int64_t L, int H, int type, T* __restrict__ out) {
  for (int64_t b = blockIdx.x; b < B; b += gridDim.x) {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const T* base = in + b * L * H + c;
      float r;
      if (type == TTB_POOL_FIRST) r = to_f(base[0]);
      else if (type == TTB_POOL_LAST) r = to_f(base[(L - 1) * H]);
      else if (type == TTB_POOL_MEAN) {
        r = 0.f;
        for (int64_t l = 0; l < L; ++l) r += to_f(base[l * H]);
        r /= (float)L;
      } else {
        r = to_f(base[0]);
        for (int64_t l = 1; l < L; ++l) r = fmaxf(r, to_f(base[l * H]));
      }
      out[b * H + c] = from_f<T>(r);
    }
  }
}

template <typename T>
__global__ void seq_pool_varlen_kernel(const T* __restrict__ in, const int32_t* __restrict__ cu, int64_t B, int H,
                                       int type, T* __restrict__ out) {
  for (int64_t b = blockIdx.x; b < B; b += gridDim.x) {
    const int64_t lo = cu[b], hi = cu[b + 1];
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float r;
      if (type == TTB_POOL_FIRST) r = to_f(in[lo * H + c]);
      else if (type == TTB_POOL_LAST) r = to_f(in[(hi - 1) * H + c]);
      else if (type == TTB_POOL_MEAN) {
        r = 0.f;
        for (int64_t l = lo; l < hi; ++l) r += to_f(in[l * H + c]);
        r /= (float)(hi - lo);
      } else {
        r = to_f(in[lo * H + c]);
        for (int64_t l = lo + 1; l < hi; ++l) r = fmaxf(r, to_f(in[l * H + c]));
      }
      out[b * H + c] = from_f<T>(r);
    }
  }
}

__global__ void prepare_masks_kernel(int64_t B, int64_t L, const int64_t* __restrict__ mask_in,
                                     int64_t* __restrict__ mask_out, int64_t* __restrict__ type_out,
                                     int64_t* __restrict__ pos_out, float* __restrict__ ext_out) {
  const int64_t n = B * L;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = mask_in ? mask_in[i] : 1;
    if (mask_out) mask_out[i] = m;
    if (type_out) type_out[i] = 0;
    if (pos_out) pos_out[i] = i % L;
    if (ext_out) ext_out[i] = -10000.0f * (1.0f - (float)m);
  }
}

// ------------------------------------------------------------------------------------------------
// Transposes between token-major [.., L, heads, d] and head-major [B, heads, L, d]; optional bias,
// optional packed<->padded mapping through cu_seqlens. One thread moves 1 element; consecutive threads
// walk d, so both sides are accessed in d-long contiguous runs.
// ------------------------------------------------------------------------------------------------
// mode 0: qkv [B,L,3,h,d] + bias -> q,k,v [B,h,L,d]     (cu == nullptr: fixed length; else packed -> padded, zero-filled)
template <typename T>
__global__ void __launch_bounds__(256)
split_add_bias_transpose_kernel(const T* __restrict__ qkv, const T* __restrict__ bias, const int32_t* __restrict__ cu,
                                int64_t B, int64_t L, int heads, int d, T* __restrict__ q, T* __restrict__ k,
                                T* __restrict__ v) {
  const int64_t H = (int64_t)heads * d;
  const int64_t n = B * L * 3 * H;  // over the padded output index space
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int dd = (int)(i % d);
    const int hh = (int)((i / d) % heads);
    const int w = (int)((i / H) % 3);
    const int64_t l = (i / (3 * H)) % L;
    const int64_t b = i / (3 * H * L);
    T* dst = (w == 0 ? q : (w == 1 ? k : v)) + ((b * heads + hh) * L + l) * d + dd;
    int64_t src_tok;
    if (cu) {
      const int64_t len = cu[b + 1] - cu[b];
      if (l >= len) { *dst = from_f<T>(0.f); continue; }
      src_tok = cu[b] + l;
    } else {
      src_tok = b * L + l;
    }
    const int64_t c = (int64_t)w * H + (int64_t)hh * d + dd;
    *dst = from_f<T>(to_f(qkv[src_tok * 3 * H + c]) + to_f(bias[c]));
  }
}

// [B,h,L,d] -> [B,L,h*d] (cu == nullptr) or padded -> packed [sumL, h*d] (cu given; index space = padded)
template <typename T>
__global__ void __launch_bounds__(256)
transpose_for_score_kernel(const T* __restrict__ in, const int32_t* __restrict__ cu, int64_t B, int64_t L, int heads,
                           int d, T* __restrict__ out) {
  const int64_t H = (int64_t)heads * d;
  const int64_t n = B * L * H;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int dd = (int)(i % d);
    const int hh = (int)((i / d) % heads);
    const int64_t l = (i / H) % L;
    const int64_t b = i / (H * L);
    int64_t dst_tok;
    if (cu) {
      if (l >= cu[b + 1] - cu[b]) continue;
      dst_tok = cu[b] + l;
    } else {
      dst_tok = b * L + l;
    }
    out[dst_tok * H + (int64_t)hh * d + dd] = in[((b * heads + hh) * L + l) * d + dd];
  }
}

// [B,L,h,d] + bias -> [B,h,L,d] (cu == nullptr) or packed [sumL,h,d] + bias -> padded, zero-filled
template <typename T>
__global__ void __launch_bounds__(256)
add_bias_transpose_kernel(const T* __restrict__ in, const T* __restrict__ bias, const int32_t* __restrict__ cu, int64_t B,
                          int64_t L, int heads, int d, T* __restrict__ out) {
  const int64_t H = (int64_t)heads * d;
  const int64_t n = B * L * H;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int dd = (int)(i % d);
    const int hh = (int)((i / d) % heads);
    const int64_t l = (i / H) % L;
    const int64_t b = i / (H * L);
    T* dst = out + ((b * heads + hh) * L + l) * d + dd;
    int64_t src_tok;
    if (cu) {
      if (l >= cu[b + 1] - cu[b]) { *dst = from_f<T>(0.f); continue; }
      src_tok = cu[b] + l;
    } else {
      src_tok = b * L + l;
    }
    const int64_t c = (int64_t)hh * d + dd;
    *dst = from_f<T>(to_f(in[src_tok * H + c]) + to_f(bias[c]));
  }
}

// ------------------------------------------------------------------------------------------------
// softmax(scores*scale + mask) over the last dim, in place; one warp per row, any row length.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
mask_softmax_kernel(T* __restrict__ scores, const float* __restrict__ mask, int64_t B, int heads, int64_t Lq,
                    int64_t Lk, float scale, int is_2d) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = B * heads * Lq;
  const int warps_total = gridDim.x * kRowsPerBlock;
  for (int64_t row = (int64_t)blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5); row < rows; row += warps_total) {
    T* s = scores + row * Lk;
    const int64_t b = row / (heads * Lq);
    const int64_t i = row % Lq;
    const float* m = mask ? mask + (is_2d ? b * Lk : (b * Lq + i) * Lk) : nullptr;
    float mx = -INFINITY;
    for (int64_t j = lane; j < Lk; j += 32) mx = fmaxf(mx, to_f(s[j]) * scale + (m ? m[j] : 0.f));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int64_t j = lane; j < Lk; j += 32) sum += expf(to_f(s[j]) * scale + (m ? m[j] : 0.f) - mx);
    const float inv = 1.0f / warp_sum(sum);
    for (int64_t j = lane; j < Lk; j += 32)
      s[j] = from_f<T>(expf(to_f(s[j]) * scale + (m ? m[j] : 0.f) - mx) * inv);
  }
}

// ------------------------------------------------------------------------------------------------
// Per-row symmetric int8 quantisation; one warp per row.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
quantize_rows_kernel(const T* __restrict__ x, int64_t M, int K, int8_t* __restrict__ xq, float* __restrict__ scale) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * kRowsPerBlock;
  for (int64_t row = (int64_t)blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5); row < M; row += warps_total) {
    const T* xr = x + row * K;
    float amax = 0.f;
    for (int c = lane; c < K; c += 32) amax = fmaxf(amax, fabsf(to_f(xr[c])));
    amax = warp_max(amax);
    const float sc = amax > 0.f ? amax / 127.0f : 1.0f;
    const float inv = __frcp_rn(sc);
    if (lane == 0) scale[row] = sc;
    for (int c = lane; c < K; c += 32) {
      float q = rintf(__fmul_rn(to_f(xr[c]), inv));
      q = fminf(fmaxf(q, -127.f), 127.f);
      xq[row * K + c] = (int8_t)q;
    }
  }
}

// The same for 16-bit rows of up to 3072 elements (K % 8 == 0): the row is loaded once with 16-byte accesses and kept
// packed in registers, two rows per warp in flight, and the int8 row leaves as 8-byte stores.
template <typename T, int ITERS>
__global__ void __launch_bounds__(kLnWarps * 32)
quantize_rows16_kernel(const T* __restrict__ x, int64_t M, int K, int8_t* __restrict__ xq, float* __restrict__ scale) {
  pdl_trigger();
  pdl_wait();
  constexpr int ROWS = 2;
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * kLnWarps;
  for (int64_t row0 = ((int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5)) * ROWS; row0 < M; row0 += warps_total * ROWS) {
    uint4 raw[ROWS][ITERS];
    float amax[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      amax[r] = 0.f;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        raw[r][it] = (row0 + r < M && col < K) ? *reinterpret_cast<const uint4*>(x + (row0 + r) * K + col) : make_uint4(0, 0, 0, 0);
        const T* h = reinterpret_cast<const T*>(&raw[r][it]);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax[r] = fmaxf(amax[r], fabsf(to_f(h[j])));
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) amax[r] = warp_max(amax[r]);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int64_t row = row0 + r;
      if (row >= M) continue;
      const float sc = amax[r] > 0.f ? amax[r] / 127.0f : 1.0f;
      const float inv = __frcp_rn(sc);
      if (lane == 0) scale[row] = sc;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        if (col < K) {
          const T* h = reinterpret_cast<const T*>(&raw[r][it]);
          uint32_t w[2] = {0u, 0u};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float q = fminf(fmaxf(rintf(__fmul_rn(to_f(h[j]), inv)), -127.f), 127.f);
            w[j >> 2] |= ((uint32_t)(int)q & 0xffu) << ((j & 3) * 8);
          }
          *reinterpret_cast<uint2*>(xq + row * K + col) = make_uint2(w[0], w[1]);
        }
      }
    }
  }
}

// Wide 16-bit rows (K % 8 == 0): two passes over the row with 16-byte accesses (the second one hits L1 / L2), so that
// nothing but the running maximum lives in registers and many warps fit an SM.
template <typename T>
__global__ void __launch_bounds__(kLnWarps * 32)
quantize_rows16_wide_kernel(const T* __restrict__ x, int64_t M, int K, int8_t* __restrict__ xq, float* __restrict__ scale) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * kLnWarps;
  for (int64_t row = (int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5); row < M; row += warps_total) {
    const T* xr = x + row * K;
    float amax = 0.f;
    for (int col = lane * 8; col < K; col += 256) {
      const uint4 q = *reinterpret_cast<const uint4*>(xr + col);
      const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(to_f(h[j])));
    }
    amax = warp_max(amax);
    const float sc = amax > 0.f ? amax / 127.0f : 1.0f;
    const float inv = __frcp_rn(sc);
    if (lane == 0) scale[row] = sc;
    for (int col = lane * 8; col < K; col += 256) {
      const uint4 q = *reinterpret_cast<const uint4*>(xr + col);
      const T* h = reinterpret_cast<const T*>(&q);
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = fminf(fmaxf(rintf(__fmul_rn(to_f(h[j]), inv)), -127.f), 127.f);
        w[j >> 2] |= ((uint32_t)(int)v & 0xffu) << ((j & 3) * 8);
      }
      *reinterpret_cast<uint2*>(xq + row * K + col) = make_uint2(w[0], w[1]);
    }
  }
}

// Rows whose maxima are known (gathered by the epilogue of the GEMM that wrote them): one streaming pass, a warp per row
// with all of the row's 16-byte loads issued before the first use. ITERS * 256 >= K.
template <typename T, int ITERS>
__global__ void __launch_bounds__(kLnWarps * 32)
quantize_rows16_given_max_kernel(const T* __restrict__ x, int64_t M, int K, const float* __restrict__ row_absmax, int8_t* __restrict__ xq,
                                 float* __restrict__ scale) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * kLnWarps;
  for (int64_t row = (int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5); row < M; row += warps_total) {
    const T* xr = x + row * K;
    uint4 raw[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int col = (it * 32 + lane) * 8;
      raw[it] = col < K ? *reinterpret_cast<const uint4*>(xr + col) : make_uint4(0, 0, 0, 0);
    }
    const float amax = row_absmax[row];
    const float sc = amax > 0.f ? amax / 127.0f : 1.0f;
    const float inv = __frcp_rn(sc);
    if (lane == 0) scale[row] = sc;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int col = (it * 32 + lane) * 8;
      if (col < K) {
        const T* h = reinterpret_cast<const T*>(&raw[it]);
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = fminf(fmaxf(rintf(__fmul_rn(to_f(h[j]), inv)), -127.f), 127.f);
          w[j >> 2] |= ((uint32_t)(int)v & 0xffu) << ((j & 3) * 8);
        }
        *reinterpret_cast<uint2*>(xq + row * K + col) = make_uint2(w[0], w[1]);
      }
    }
  }
}

// LayerNorm of 16-bit rows that also leaves the int8 form of its output (per-row symmetric, the quantiser above applied
// to the rounded 16-bit values, so the result is the same as running the two kernels one after the other): the input of
// an int8 Linear is produced where it is computed instead of by another pass over the activations.
template <typename T, int ITERS, int ROWS>
__global__ void __launch_bounds__(kLnWarps * 32)
layernorm16_quant_kernel(const T* x, const T* __restrict__ gamma, const T* __restrict__ beta, T* out, int8_t* __restrict__ xq,
                         float* __restrict__ scale, int64_t M, int N, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * kLnWarps;
  for (int64_t row0 = ((int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5)) * ROWS; row0 < M; row0 += warps_total * ROWS) {
    uint4 raw[ROWS][ITERS];
    float mean[ROWS], rstd[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      float sum = 0.f, sq = 0.f;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        raw[r][it] = (row0 + r < M && col < N) ? *reinterpret_cast<const uint4*>(x + (row0 + r) * N + col) : make_uint4(0, 0, 0, 0);
        const T* h = reinterpret_cast<const T*>(&raw[r][it]);
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float f = to_f(h[j]); sum += f; sq = fmaf(f, f, sq); }
      }
      mean[r] = sum;
      rstd[r] = sq;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {  // from here on mean[] holds the shift -mean * rstd
      const float sum = warp_sum(mean[r]), sq = warp_sum(rstd[r]);
      ln_row_params(sum, sq, 1.0f / (float)N, eps, rstd[r], mean[r]);
    }
    // normalise in place: the packed registers now hold the rounded 16-bit output, which is also what gets quantised
    float amax[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) amax[r] = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int col = (it * 32 + lane) * 8;
      if (col < N) {
        const uint4 gq = *reinterpret_cast<const uint4*>(gamma + col), bq = *reinterpret_cast<const uint4*>(beta + col);
        const T* g = reinterpret_cast<const T*>(&gq);
        const T* b = reinterpret_cast<const T*>(&bq);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          T* h = reinterpret_cast<T*>(&raw[r][it]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            h[j] = from_f<T>(ln_value(to_f(h[j]), rstd[r], mean[r], to_f(g[j]), to_f(b[j])));
            amax[r] = fmaxf(amax[r], fabsf(to_f(h[j])));
          }
          if (row0 + r < M) *reinterpret_cast<uint4*>(out + (row0 + r) * N + col) = raw[r][it];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int64_t row = row0 + r;
      const float am = warp_max(amax[r]);
      if (row >= M) continue;
      const float sc = am > 0.f ? am / 127.0f : 1.0f;
      const float inv = __frcp_rn(sc);
      if (lane == 0) scale[row] = sc;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int col = (it * 32 + lane) * 8;
        if (col < N) {
          const T* h = reinterpret_cast<const T*>(&raw[r][it]);
          uint32_t w[2] = {0u, 0u};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float v = fminf(fmaxf(rintf(__fmul_rn(to_f(h[j]), inv)), -127.f), 127.f);
            w[j >> 2] |= ((uint32_t)(int)v & 0xffu) << ((j & 3) * 8);
          }
          *reinterpret_cast<uint2*>(xq + row * N + col) = make_uint2(w[0], w[1]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Per-tensor affine 7-bit quantisation of activations (torch's dynamic quantisation with reduce_range): a running
// minimum / maximum over the whole tensor, then q = clamp(rint(zp + x * (1 / scale)), 0, 127).
// qparams: [0] scale, [1] zero point (as a float), [2] / [3] minimum / maximum as order-preserving integers.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ int float_to_ordered(float f) {
  const int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_to_float(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__global__ void affine_range_init_kernel(float* qparams) {
  // the quantised range always contains zero, so zero is the starting point of both ends
  reinterpret_cast<int*>(qparams)[2] = float_to_ordered(0.f);
  reinterpret_cast<int*>(qparams)[3] = float_to_ordered(0.f);
}

template <typename T>
__global__ void __launch_bounds__(256) affine_range_kernel(const T* __restrict__ x, int64_t n, float* qparams) {
  float mn = 0.f, mx = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = to_f(x[i]);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  mn = -warp_max(-mn);
  if ((threadIdx.x & 31) == 0) {
    atomicMin(reinterpret_cast<int*>(qparams) + 2, float_to_ordered(mn));
    atomicMax(reinterpret_cast<int*>(qparams) + 3, float_to_ordered(mx));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) affine_quantize_kernel(const T* __restrict__ x, int64_t n, int8_t* __restrict__ xq, float* qparams) {
  const double mn = (double)ordered_to_float(reinterpret_cast<const int*>(qparams)[2]);
  const double mx = (double)ordered_to_float(reinterpret_cast<const int*>(qparams)[3]);
  double scale = (mx - mn) / 127.0;
  if ((float)scale == 0.f || isinf(1.0f / (float)scale)) scale = 0.1;
  const double zp_from_min = 0.0 - mn / scale, zp_from_max = 127.0 - mx / scale;
  const double err_min = 0.0 - fabs(mn / scale), err_max = 127.0 - fabs(mx / scale);
  double zpd = err_min < err_max ? zp_from_min : zp_from_max;
  zpd = zpd < 0.0 ? 0.0 : (zpd > 127.0 ? 127.0 : rint(zpd));
  const float fscale = (float)scale, inv = 1.0f / fscale, zp = (float)zpd;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    qparams[0] = fscale;
    qparams[1] = zp;
  }
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    // two separately rounded operations, as the CPU code does them (no fused multiply-add)
    const float q = rintf(__fadd_rn(zp, __fmul_rn(to_f(x[i]), inv)));
    xq[i] = (int8_t)fminf(fmaxf(q, 0.f), 127.f);
  }
}

}  // namespace

// =================================================================================================
// C ABI
// =================================================================================================
extern "C" int ttb_add_bias_layernorm(ttb_ctx* ctx, int dtype, void* out, const void* input, const void* bias,
                                      const void* gamma, const void* beta, int64_t M, int64_t N, float eps) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0, "add_bias_layernorm: bad shape M=%lld N=%lld", (long long)M, (long long)N);
  TTB_REQUIRE(ctx, M == 0 || (out && input && bias && gamma && beta), "add_bias_layernorm: null pointer");
  DeviceGuard g(ctx->device);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     return (launch_layernorm<T, T, true>(ctx, (const T*)out, (const T*)input, (const T*)bias, (const T*)gamma,
                                                          (const T*)beta, (T*)out, nullptr, nullptr, M, N, eps)));
  return TTB_OK;
}

extern "C" int ttb_layernorm(ttb_ctx* ctx, int dtype, const void* in, void* out, const void* gamma, const void* beta,
                             int64_t M, int64_t N, float eps) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0, "layernorm: bad shape");
  TTB_REQUIRE(ctx, M == 0 || (in && out && gamma && beta), "layernorm: null pointer");
  DeviceGuard g(ctx->device);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     return (launch_layernorm<T, T, false>(ctx, (const T*)in, nullptr, nullptr, (const T*)gamma,
                                                           (const T*)beta, (T*)out, nullptr, nullptr, M, N, eps)));
  return TTB_OK;
}

extern "C" int ttb_layernorm_planes(ttb_ctx* ctx, int in_dtype, int out_dtype, const void* in, void* out, void* out_lo, float* out_f32,
                                    const void* gamma, const void* beta, int64_t M, int64_t N, float eps) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0, "layernorm_planes: bad shape");
  TTB_REQUIRE(ctx, M == 0 || (in && out && gamma && beta), "layernorm_planes: null pointer");
  TTB_REQUIRE(ctx, out_dtype == TTB_F16 || out_dtype == TTB_BF16, "layernorm_planes: the output dtype must be F16 or BF16");
  TTB_REQUIRE(ctx, in_dtype == out_dtype || in_dtype == TTB_F32, "layernorm_planes: the input is of the output dtype or F32");
  DeviceGuard g(ctx->device);
  if (out_dtype == TTB_F16) {
    using T = __half;
    if (in_dtype == TTB_F32)
      return launch_layernorm<float, T, false>(ctx, (const float*)in, nullptr, nullptr, (const T*)gamma, (const T*)beta, (T*)out, (T*)out_lo, out_f32, M, N, eps);
    return launch_layernorm<T, T, false>(ctx, (const T*)in, nullptr, nullptr, (const T*)gamma, (const T*)beta, (T*)out, (T*)out_lo, out_f32, M, N, eps);
  }
  using T = __nv_bfloat16;
  if (in_dtype == TTB_F32)
    return launch_layernorm<float, T, false>(ctx, (const float*)in, nullptr, nullptr, (const T*)gamma, (const T*)beta, (T*)out, (T*)out_lo, out_f32, M, N, eps);
  return launch_layernorm<T, T, false>(ctx, (const T*)in, nullptr, nullptr, (const T*)gamma, (const T*)beta, (T*)out, (T*)out_lo, out_f32, M, N, eps);
}

extern "C" int ttb_add_bias_act(ttb_ctx* ctx, int dtype, void* out, const void* bias, int64_t M, int64_t N, int act) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0, "add_bias_act: bad shape");
  TTB_REQUIRE(ctx, act >= 0 && act <= 2, "add_bias_act: unknown activation %d", act);
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, out && bias, "add_bias_act: null pointer");
  DeviceGuard g(ctx->device);
  const bool vec = N % 8 == 0 && (reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) % 16 == 0;
  const int grid = grid_for(vec ? M * N / 8 : M * N, 256, ctx->sm_count);
#define ACT_CASE(A)                                                                                    \
  if (vec) add_bias_act_kernel<T, A, true><<<grid, 256, 0, ctx->stream>>>((T*)out, (const T*)bias, M, (int)N); \
  else add_bias_act_kernel<T, A, false><<<grid, 256, 0, ctx->stream>>>((T*)out, (const T*)bias, M, (int)N)
  TTB_DISPATCH_FLOAT(ctx, dtype, T, {
    if (act == TTB_ACT_GELU) { ACT_CASE(TTB_ACT_GELU); }
    else if (act == TTB_ACT_TANH) { ACT_CASE(TTB_ACT_TANH); }
    else { ACT_CASE(TTB_ACT_RELU); }
  });
#undef ACT_CASE
  return launched(ctx, "add_bias_act");
}

extern "C" int ttb_add_bias(ttb_ctx* ctx, int dtype, void* out, const void* bias, int64_t M, int64_t N) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0, "add_bias: bad shape");
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, out && bias, "add_bias: null pointer");
  DeviceGuard g(ctx->device);
  const int grid = grid_for(M * N, 256, ctx->sm_count);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (add_bias_kernel<T, false><<<grid, 256, 0, ctx->stream>>>((const T*)out, nullptr, (const T*)bias, (T*)out, M, (int)N)));
  return launched(ctx, "add_bias");
}

extern "C" int ttb_add_input_bias(ttb_ctx* ctx, int dtype, const void* in1, const void* in2, const void* bias,
                                  int64_t M, int64_t N, void* out) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0, "add_input_bias: bad shape");
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, in1 && in2 && bias && out, "add_input_bias: null pointer");
  DeviceGuard g(ctx->device);
  const int grid = grid_for(M * N, 256, ctx->sm_count);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (add_bias_kernel<T, true><<<grid, 256, 0, ctx->stream>>>((const T*)in1, (const T*)in2, (const T*)bias, (T*)out, M, (int)N)));
  return launched(ctx, "add_input_bias");
}

extern "C" int ttb_lookup_embedding(ttb_ctx* ctx, int dtype, void* out, const void* table, const int64_t* ids,
                                    int64_t n_ids, int64_t hidden, int64_t vocab, int add) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, n_ids >= 0 && hidden > 0 && vocab > 0, "lookup_embedding: bad shape");
  if (n_ids == 0) return TTB_OK;
  TTB_REQUIRE(ctx, out && table && ids, "lookup_embedding: null pointer");
  DeviceGuard g(ctx->device);
  const int grid = (int)(n_ids < (int64_t)ctx->sm_count * 16 ? n_ids : (int64_t)ctx->sm_count * 16);
  const int block = hidden >= 256 ? 256 : 128;
  TTB_DISPATCH_FLOAT(ctx, dtype, T, {
    if (add) lookup_kernel<T, true><<<grid, block, 0, ctx->stream>>>((T*)out, (const T*)table, ids, n_ids, (int)hidden, vocab, ctx->d_status);
    else lookup_kernel<T, false><<<grid, block, 0, ctx->stream>>>((T*)out, (const T*)table, ids, n_ids, (int)hidden, vocab, ctx->d_status);
  });
  return launched(ctx, "lookup_embedding");
}

extern "C" int ttb_embedding_ln(ttb_ctx* ctx, int dtype, const int64_t* ids, const int64_t* position_ids,
                                const int64_t* token_type_ids, const int32_t* cu_seqlens, int64_t B, int64_t seq_len,
                                int64_t n_tokens, const void* word, const void* position, const void* token_type,
                                const void* gamma, const void* beta, int64_t hidden, int64_t vocab,
                                int64_t n_positions, int64_t n_types, float eps, void* out) {
  return ttb_embedding_ln_planes(ctx, dtype, ids, position_ids, token_type_ids, cu_seqlens, B, seq_len, n_tokens, word, position, token_type,
                                 gamma, beta, hidden, vocab, n_positions, n_types, eps, out, nullptr, nullptr);
}

extern "C" int ttb_embedding_ln_planes(ttb_ctx* ctx, int dtype, const int64_t* ids, const int64_t* position_ids,
                                       const int64_t* token_type_ids, const int32_t* cu_seqlens, int64_t B, int64_t seq_len,
                                       int64_t n_tokens, const void* word, const void* position, const void* token_type,
                                       const void* gamma, const void* beta, int64_t hidden, int64_t vocab, int64_t n_positions,
                                       int64_t n_types, float eps, void* out, void* out_lo, float* out_f32) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, n_tokens >= 0 && hidden > 0 && vocab > 0 && n_positions > 0 && n_types > 0, "embedding_ln: bad shape");
  if (n_tokens == 0) return TTB_OK;
  TTB_REQUIRE(ctx, ids && word && position && token_type && gamma && beta && out, "embedding_ln: null pointer");
  TTB_REQUIRE(ctx, position_ids || cu_seqlens || seq_len > 0, "embedding_ln: need position_ids, cu_seqlens or seq_len");
  TTB_REQUIRE(ctx, !cu_seqlens || B > 0, "embedding_ln: cu_seqlens needs B > 0");
  DeviceGuard g(ctx->device);
  const int grid = grid_for(n_tokens, kRowsPerBlock, ctx->sm_count);
  const bool all16 = ((reinterpret_cast<uintptr_t>(word) | reinterpret_cast<uintptr_t>(position) | reinterpret_cast<uintptr_t>(token_type) |
                       reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta) | reinterpret_cast<uintptr_t>(out) |
                       reinterpret_cast<uintptr_t>(out_lo) | reinterpret_cast<uintptr_t>(out_f32)) & 15) == 0;
  if ((dtype == TTB_F16 || dtype == TTB_BF16) && hidden % 8 == 0 && hidden <= 1024 && all16) {
#define EMB16(T, IT)                                                                                                                         \
  launch_pdl(embedding_ln16_kernel<T, IT>, dim3(grid), dim3(kRowsPerBlock * 32), 0, ctx->stream, ids, position_ids, token_type_ids, cu_seqlens,  \
             (int)B, (int)(seq_len > 0 ? seq_len : 1), n_tokens, (const T*)word, (const T*)position, (const T*)token_type, (const T*)gamma,       \
             (const T*)beta, (int)hidden, vocab, n_positions, n_types, eps, (T*)out, (T*)out_lo, out_f32, ctx->d_status)
#define EMB16_PICK(T)                    \
  do {                                   \
    if (hidden <= 256) EMB16(T, 1);      \
    else if (hidden <= 512) EMB16(T, 2); \
    else if (hidden <= 768) EMB16(T, 3); \
    else EMB16(T, 4);                    \
  } while (0)
    if (dtype == TTB_F16) EMB16_PICK(__half);
    else EMB16_PICK(__nv_bfloat16);
#undef EMB16_PICK
#undef EMB16
    return launched(ctx, "embedding_ln");
  }
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (embedding_ln_kernel<T><<<grid, kRowsPerBlock * 32, 0, ctx->stream>>>(
                         ids, position_ids, token_type_ids, cu_seqlens, (int)B, (int)(seq_len > 0 ? seq_len : 1), n_tokens,
                         (const T*)word, (const T*)position, (const T*)token_type, (const T*)gamma, (const T*)beta,
                         (int)hidden, vocab, n_positions, n_types, eps, (T*)out, (T*)out_lo, out_f32, ctx->d_status)));
  return launched(ctx, "embedding_ln");
}

extern "C" int ttb_seq_pool(ttb_ctx* ctx, int dtype, const void* in, int64_t B, int64_t L, int64_t H, int pool_type,
                            void* out) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, B >= 0 && L > 0 && H > 0, "seq_pool: bad shape");
  TTB_REQUIRE(ctx, pool_type >= 0 && pool_type <= 3, "seq_pool: unknown pool type %d", pool_type);
  if (B == 0) return TTB_OK;
  TTB_REQUIRE(ctx, in && out, "seq_pool: null pointer");
  DeviceGuard g(ctx->device);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (seq_pool_kernel<T><<<(int)(B < 65535 ? B : 65535), 256, 0, ctx->stream>>>((const T*)in, B, L, (int)H, pool_type, (T*)out)));
  return launched(ctx, "seq_pool");
}

extern "C" int ttb_seq_pool_varlen(ttb_ctx* ctx, int dtype, const void* in, const int32_t* cu_seqlens, int64_t B,
                                   int64_t H, int pool_type, void* out) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, B >= 0 && H > 0, "seq_pool_varlen: bad shape");
  TTB_REQUIRE(ctx, pool_type >= 0 && pool_type <= 3, "seq_pool_varlen: unknown pool type %d", pool_type);
  if (B == 0) return TTB_OK;
  TTB_REQUIRE(ctx, in && out && cu_seqlens, "seq_pool_varlen: null pointer");
  DeviceGuard g(ctx->device);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (seq_pool_varlen_kernel<T><<<(int)(B < 65535 ? B : 65535), 256, 0, ctx->stream>>>((const T*)in, cu_seqlens, B, (int)H, pool_type, (T*)out)));
  return launched(ctx, "seq_pool_varlen");
}

extern "C" int ttb_prepare_bert_masks(ttb_ctx* ctx, int64_t B, int64_t L, const int64_t* att_mask_in,
                                      int64_t* att_mask_out, int64_t* token_type_out, int64_t* position_ids_out,
                                      float* extended_out) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, B >= 0 && L >= 0, "prepare_bert_masks: bad shape");
  if (B * L == 0) return TTB_OK;
  DeviceGuard g(ctx->device);
  prepare_masks_kernel<<<grid_for(B * L, 256, ctx->sm_count), 256, 0, ctx->stream>>>(B, L, att_mask_in, att_mask_out, token_type_out,
                                                                                      position_ids_out, extended_out);
  return launched(ctx, "prepare_bert_masks");
}

static int check_transpose_args(ttb_ctx* ctx, const char* what, int64_t B, int64_t L, int64_t heads, int64_t d) {
  TTB_REQUIRE(ctx, B >= 0 && L >= 0 && heads > 0 && d > 0, "%s: bad shape B=%lld L=%lld heads=%lld d=%lld", what,
              (long long)B, (long long)L, (long long)heads, (long long)d);
  return TTB_OK;
}

extern "C" int ttb_split_add_bias_transpose(ttb_ctx* ctx, int dtype, const void* qkv, const void* bias, int64_t B,
                                            int64_t L, int64_t heads, int64_t d, void* q, void* k, void* v) {
  return ttb_split_add_bias_transpose_pad(ctx, dtype, qkv, bias, nullptr, B, L, heads, d, q, k, v);
}

extern "C" int ttb_split_add_bias_transpose_pad(ttb_ctx* ctx, int dtype, const void* qkv, const void* bias,
                                                const int32_t* cu_seqlens, int64_t B, int64_t maxL, int64_t heads,
                                                int64_t d, void* q, void* k, void* v) {
  if (!ctx) return TTB_ERR_INVALID;
  int s = check_transpose_args(ctx, "split_add_bias_transpose", B, maxL, heads, d);
  if (s) return s;
  if (B * maxL == 0) return TTB_OK;
  TTB_REQUIRE(ctx, qkv && bias && q && k && v, "split_add_bias_transpose: null pointer");
  DeviceGuard g(ctx->device);
  const int grid = grid_for(B * maxL * 3 * heads * d, 256, ctx->sm_count);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (split_add_bias_transpose_kernel<T><<<grid, 256, 0, ctx->stream>>>((const T*)qkv, (const T*)bias, cu_seqlens, B, maxL,
                                                                                      (int)heads, (int)d, (T*)q, (T*)k, (T*)v)));
  return launched(ctx, "split_add_bias_transpose");
}

extern "C" int ttb_transpose_for_score(ttb_ctx* ctx, int dtype, const void* in, int64_t B, int64_t heads, int64_t L,
                                       int64_t d, void* out) {
  return ttb_transpose_for_score_pad(ctx, dtype, in, nullptr, B, L, heads, d, out);
}

extern "C" int ttb_transpose_for_score_pad(ttb_ctx* ctx, int dtype, const void* in, const int32_t* cu_seqlens,
                                           int64_t B, int64_t maxL, int64_t heads, int64_t d, void* out) {
  if (!ctx) return TTB_ERR_INVALID;
  int s = check_transpose_args(ctx, "transpose_for_score", B, maxL, heads, d);
  if (s) return s;
  if (B * maxL == 0) return TTB_OK;
  TTB_REQUIRE(ctx, in && out, "transpose_for_score: null pointer");
  DeviceGuard g(ctx->device);
  const int grid = grid_for(B * maxL * heads * d, 256, ctx->sm_count);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (transpose_for_score_kernel<T><<<grid, 256, 0, ctx->stream>>>((const T*)in, cu_seqlens, B, maxL, (int)heads, (int)d, (T*)out)));
  return launched(ctx, "transpose_for_score");
}

extern "C" int ttb_add_bias_transpose_for_score(ttb_ctx* ctx, int dtype, const void* in, const void* bias, int64_t B,
                                                int64_t L, int64_t heads, int64_t d, void* out) {
  return ttb_add_bias_transpose_for_score_pad(ctx, dtype, in, bias, nullptr, B, L, heads, d, out);
}

extern "C" int ttb_add_bias_transpose_for_score_pad(ttb_ctx* ctx, int dtype, const void* in, const void* bias,
                                                    const int32_t* cu_seqlens, int64_t B, int64_t maxL, int64_t heads,
                                                    int64_t d, void* out) {
  if (!ctx) return TTB_ERR_INVALID;
  int s = check_transpose_args(ctx, "add_bias_transpose_for_score", B, maxL, heads, d);
  if (s) return s;
  if (B * maxL == 0) return TTB_OK;
  TTB_REQUIRE(ctx, in && bias && out, "add_bias_transpose_for_score: null pointer");
  DeviceGuard g(ctx->device);
  const int grid = grid_for(B * maxL * heads * d, 256, ctx->sm_count);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (add_bias_transpose_kernel<T><<<grid, 256, 0, ctx->stream>>>((const T*)in, (const T*)bias, cu_seqlens, B, maxL, (int)heads,
                                                                                (int)d, (T*)out)));
  return launched(ctx, "add_bias_transpose_for_score");
}

extern "C" int ttb_mask_softmax(ttb_ctx* ctx, int dtype, void* scores, const float* mask, int64_t B, int64_t heads,
                                int64_t Lq, int64_t Lk, float scale, int mask_is_2d) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, B >= 0 && heads > 0 && Lq >= 0 && Lk > 0, "mask_softmax: bad shape");
  if (B * Lq == 0) return TTB_OK;
  TTB_REQUIRE(ctx, scores, "mask_softmax: null pointer");
  DeviceGuard g(ctx->device);
  const int grid = grid_for(B * heads * Lq, kRowsPerBlock, ctx->sm_count);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (mask_softmax_kernel<T><<<grid, kRowsPerBlock * 32, 0, ctx->stream>>>((T*)scores, mask, B, (int)heads, Lq, Lk, scale, mask_is_2d)));
  return launched(ctx, "mask_softmax");
}

extern "C" int ttb_quantize_rows_int8(ttb_ctx* ctx, int dtype, const void* x, int64_t M, int64_t K, int8_t* xq,
                                      float* row_scale) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && K > 0, "quantize_rows_int8: bad shape");
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, x && xq && row_scale, "quantize_rows_int8: null pointer");
  DeviceGuard g(ctx->device);
  const bool aligned = K % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xq)) & 15) == 0;
  if ((dtype == TTB_F16 || dtype == TTB_BF16) && aligned && K > 1024) {
    const int gridw = grid_for(M, kLnWarps, ctx->sm_count);
    if (dtype == TTB_F16)
      launch_pdl(quantize_rows16_wide_kernel<__half>, dim3(gridw), dim3(kLnWarps * 32), 0, ctx->stream, (const __half*)x, M, (int)K, xq, row_scale);
    else
      launch_pdl(quantize_rows16_wide_kernel<__nv_bfloat16>, dim3(gridw), dim3(kLnWarps * 32), 0, ctx->stream, (const __nv_bfloat16*)x, M, (int)K, xq,
                 row_scale);
    return launched(ctx, "quantize_rows_int8");
  }
  if ((dtype == TTB_F16 || dtype == TTB_BF16) && aligned) {
    const int grid16 = grid_for((M + 1) / 2, kLnWarps, ctx->sm_count);
#define Q16_CASE(T, IT) launch_pdl(quantize_rows16_kernel<T, IT>, dim3(grid16), dim3(kLnWarps * 32), 0, ctx->stream, (const T*)x, M, (int)K, xq, row_scale)
#define Q16_PICK(T)                      \
  do {                                   \
    if (K <= 256) Q16_CASE(T, 1);        \
    else if (K <= 768) Q16_CASE(T, 3);   \
    else Q16_CASE(T, 4);                 \
  } while (0)
    if (dtype == TTB_F16) Q16_PICK(__half);
    else Q16_PICK(__nv_bfloat16);
#undef Q16_PICK
#undef Q16_CASE
    return launched(ctx, "quantize_rows_int8");
  }
  const int grid = grid_for(M, kRowsPerBlock, ctx->sm_count);
  TTB_DISPATCH_FLOAT(ctx, dtype, T,
                     (quantize_rows_kernel<T><<<grid, kRowsPerBlock * 32, 0, ctx->stream>>>((const T*)x, M, (int)K, xq, row_scale)));
  return launched(ctx, "quantize_rows_int8");
}

extern "C" int ttb_quantize_rows_int8_given_max(ttb_ctx* ctx, int dtype, const void* x, int64_t M, int64_t K, const float* row_absmax,
                                                int8_t* xq, float* row_scale) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && K > 0, "quantize_rows_int8_given_max: bad shape");
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, x && xq && row_scale && row_absmax, "quantize_rows_int8_given_max: null pointer");
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "quantize_rows_int8_given_max: F16 or BF16 rows");
  TTB_REQUIRE(ctx, K % 8 == 0 && K <= 4096 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xq)) & 15) == 0,
              "quantize_rows_int8_given_max: K %% 8 == 0, K <= 4096 and 16-byte aligned pointers (K = %lld)", (long long)K);
  DeviceGuard g(ctx->device);
  const int grid = grid_for(M, kLnWarps, ctx->sm_count);
#define QG_CASE(T, IT) \
  launch_pdl(quantize_rows16_given_max_kernel<T, IT>, dim3(grid), dim3(kLnWarps * 32), 0, ctx->stream, (const T*)x, M, (int)K, row_absmax, xq, row_scale)
#define QG_PICK(T)                       \
  do {                                   \
    if (K <= 1024) QG_CASE(T, 4);        \
    else if (K <= 2048) QG_CASE(T, 8);   \
    else if (K <= 3072) QG_CASE(T, 12);  \
    else QG_CASE(T, 16);                 \
  } while (0)
  if (dtype == TTB_F16) QG_PICK(__half);
  else QG_PICK(__nv_bfloat16);
#undef QG_PICK
#undef QG_CASE
  return launched(ctx, "quantize_rows_int8_given_max");
}

extern "C" int ttb_quantize_tensor_affine(ttb_ctx* ctx, int dtype, const void* x, int64_t M, int64_t K, int8_t* xq, float* qparams) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && K > 0, "quantize_tensor_affine: bad shape");
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, x && xq && qparams, "quantize_tensor_affine: null pointer");
  DeviceGuard g(ctx->device);
  const int64_t n = M * K;
  const int64_t want = (n + 255) / 256;
  const int grid = (int)(want < (int64_t)ctx->sm_count * 8 ? want : (int64_t)ctx->sm_count * 8);
  affine_range_init_kernel<<<1, 1, 0, ctx->stream>>>(qparams);
  TTB_DISPATCH_FLOAT(ctx, dtype, T, {
    affine_range_kernel<T><<<grid, 256, 0, ctx->stream>>>((const T*)x, n, qparams);
    affine_quantize_kernel<T><<<grid, 256, 0, ctx->stream>>>((const T*)x, n, xq, qparams);
  });
  ctx->launches.fetch_add(2);
  return launched(ctx, "quantize_tensor_affine");
}

namespace {
// Up to this many lengths travel inside the kernel's parameter block: no staging copy and nothing for the host to wait for.
constexpr int kLensInParams = 960;
struct LensParam {
  int32_t v[kLensInParams];
};
__global__ void cu_seqlens_from_params_kernel(const LensParam lens, int B, int32_t* __restrict__ cu) {
  // one warp: an inclusive scan over chunks of 32 lengths, carrying the running total
  const int lane = threadIdx.x;
  int carry = 0;
  if (lane == 0) cu[0] = 0;
  for (int base = 0; base < B; base += 32) {
    int v = (base + lane < B) ? lens.v[base + lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    if (base + lane < B) cu[base + lane + 1] = carry + v;
    carry += __shfl_sync(0xffffffffu, v, 31);
  }
}
}  // namespace

extern "C" int ttb_layernorm_quant_int8(ttb_ctx* ctx, int dtype, const void* in, void* out, int8_t* xq, float* row_scale, const void* gamma,
                                        const void* beta, int64_t M, int64_t N, float eps) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0, "layernorm_quant_int8: bad shape");
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, in && out && xq && row_scale && gamma && beta, "layernorm_quant_int8: null pointer");
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "layernorm_quant_int8: dtype must be F16 or BF16");
  const bool aligned = N % 8 == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(xq) |
                                       reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15) == 0;
  if (!aligned || N > 1024) {  // shapes without a fused kernel: the two kernels one after the other give the same result
    int s = ttb_layernorm(ctx, dtype, in, out, gamma, beta, M, N, eps);
    if (s != TTB_OK) return s;
    return ttb_quantize_rows_int8(ctx, dtype, out, M, N, xq, row_scale);
  }
  DeviceGuard g(ctx->device);
  // few rows (a single short request): one row per warp, so that the kernel is spread over more SMs
  const bool few = M <= 8 * (int64_t)ctx->sm_count;
  const int grid = grid_for(few ? M : (M + 1) / 2, kLnWarps, ctx->sm_count);
#define LNQ_CASE(T, IT)                                                                                                                 \
  do {                                                                                                                                  \
    if (few)                                                                                                                            \
      launch_pdl(layernorm16_quant_kernel<T, IT, 1>, dim3(grid), dim3(kLnWarps * 32), 0, ctx->stream, (const T*)in, (const T*)gamma,    \
                 (const T*)beta, (T*)out, xq, row_scale, M, (int)N, eps);                                                               \
    else                                                                                                                                \
      launch_pdl(layernorm16_quant_kernel<T, IT, 2>, dim3(grid), dim3(kLnWarps * 32), 0, ctx->stream, (const T*)in, (const T*)gamma,    \
                 (const T*)beta, (T*)out, xq, row_scale, M, (int)N, eps);                                                               \
  } while (0)
#define LNQ_PICK(T)                     \
  do {                                  \
    if (N <= 256) LNQ_CASE(T, 1);       \
    else if (N <= 512) LNQ_CASE(T, 2);  \
    else if (N <= 768) LNQ_CASE(T, 3);  \
    else LNQ_CASE(T, 4);                \
  } while (0)
  if (dtype == TTB_F16) LNQ_PICK(__half);
  else LNQ_PICK(__nv_bfloat16);
#undef LNQ_PICK
#undef LNQ_CASE
  return launched(ctx, "layernorm_quant_int8");
}

extern "C" int ttb_build_cu_seqlens(ttb_ctx* ctx, const int64_t* host_seq_lens, int64_t B, int32_t* cu_dev) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, B >= 0 && (B == 0 || host_seq_lens) && cu_dev, "build_cu_seqlens: bad arguments");
  if (B <= kLensInParams) {
    LensParam lp;
    int64_t total = 0;
    for (int64_t b = 0; b < B; ++b) {
      TTB_REQUIRE(ctx, host_seq_lens[b] >= 0, "build_cu_seqlens: negative length at %lld", (long long)b);
      total += host_seq_lens[b];
      TTB_REQUIRE(ctx, total <= INT32_MAX, "build_cu_seqlens: more than 2^31 tokens");
      lp.v[b] = (int32_t)host_seq_lens[b];
    }
    DeviceGuard g(ctx->device);
    cu_seqlens_from_params_kernel<<<1, 32, 0, ctx->stream>>>(lp, (int)B, cu_dev);
    return launched(ctx, "build_cu_seqlens");
  }
  std::vector<int32_t> cu((size_t)B + 1, 0);
  for (int64_t b = 0; b < B; ++b) {
    TTB_REQUIRE(ctx, host_seq_lens[b] >= 0, "build_cu_seqlens: negative length at %lld", (long long)b);
    int64_t next = (int64_t)cu[b] + host_seq_lens[b];
    TTB_REQUIRE(ctx, next <= INT32_MAX, "build_cu_seqlens: more than 2^31 tokens");
    cu[b + 1] = (int32_t)next;
  }
  DeviceGuard g(ctx->device);
  // pageable source: the copy has completed from the host's view when the call returns
  TTB_CUDA(ctx, cudaMemcpyAsync(cu_dev, cu.data(), cu.size() * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
  TTB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return TTB_OK;
}
