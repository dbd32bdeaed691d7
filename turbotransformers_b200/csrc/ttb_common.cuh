// Shared internals of libttb: the context object, error plumbing and dtype helpers.
#pragma once
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "ttb.h"

struct ttb_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  cudaMemPool_t pool = nullptr;
  bool owns_pool = false;
  int* d_status = nullptr;  // device word kernels write instead of trapping
  int* h_status = nullptr;  // pinned mirror
  int sm_count = 148;
  std::string last_error;
  std::mutex mu;            // guards last_error and pool statistics
  size_t in_use = 0, high_water = 0, limit = 0;
  uint64_t n_allocs = 0;
  std::atomic<uint64_t> launches{0};
  std::unordered_map<void*, size_t> live;
  // arena mode (ttb_arena_begin / ttb_arena_end): allocations at increasing offsets of one reserved buffer. Every
  // begin reserves a buffer of its own; after end it belongs to the caller until ttb_arena_release.
  char* arena = nullptr;  // the active arena
  size_t arena_size = 0, arena_off = 0, arena_peak = 0;
  bool arena_active = false;
  std::vector<std::pair<char*, size_t>> arenas;  // every reserved buffer not yet released (the active one included)
  uint64_t bytes_allocated_total = 0;  // sum of all ttb_alloc sizes so far
  // workspace of the GEMM kernels whose epilogue is a LayerNorm: per-row partial sums and per-row-block counters. Owned by
  // the context (not the pool): the counters must be zero between launches, which the kernels themselves see to.
  void* ln_ws = nullptr;
  size_t ln_ws_rows = 0;  // rows the workspace is sized for
};

namespace ttb {

inline int fail(ttb_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) {
    std::lock_guard<std::mutex> g(ctx->mu);
    ctx->last_error = buf;
  }
  return code;
}

#define TTB_CUDA(ctx, expr)                                                                     \
  do {                                                                                          \
    cudaError_t e__ = (expr);                                                                   \
    if (e__ != cudaSuccess)                                                                     \
      return ::ttb::fail(ctx, TTB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                         __FILE__, __LINE__);                                                   \
  } while (0)

#define TTB_REQUIRE(ctx, cond, ...)                                    \
  do {                                                                 \
    if (!(cond)) return ::ttb::fail(ctx, TTB_ERR_INVALID, __VA_ARGS__); \
  } while (0)

// Called after every kernel launch: counts it and surfaces launch-configuration errors.
inline int launched(ttb_ctx* ctx, const char* what) {
  ctx->launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ctx, TTB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  return TTB_OK;
}

// ---- programmatic dependent launch ------------------------------------------------------------------------------
// A kernel launched through launch_pdl may be scheduled before the kernel ahead of it in the stream has finished: its
// CTAs run their set-up (barrier initialisation, tensor-memory allocation, descriptor fetches) in the shadow of that
// kernel's tail. Such a kernel must execute pdl_wait() in EVERY CTA before it reads or writes global memory (and before
// any early return, so that "this grid is complete" keeps implying "everything ahead of it in the stream is complete");
// pdl_trigger() lets the grid behind it start its own set-up. Set TTB_PDL=0 to launch everything fully serialised.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("TTB_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

inline size_t dtype_size(int dt) {
  switch (dt) {
    case TTB_F32: return 4;
    case TTB_F16: return 2;
    case TTB_BF16: return 2;
    case TTB_I8: return 1;
  }
  return 0;
}

// ---- device-side scalar conversion -------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A group of 8 consecutive elements moved with 16-byte (or 2x16-byte for fp32) accesses.
template <typename T> struct Vec8 {
  float v[8];
  __device__ __forceinline__ void load(const T* p);
  __device__ __forceinline__ void store(T* p) const;
};
template <> __device__ __forceinline__ void Vec8<float>::load(const float* p) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void Vec8<float>::store(float* p) const {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void Vec8<__half>::load(const __half* p) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void Vec8<__half>::store(__half* p) const {
  uint4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}
template <> __device__ __forceinline__ void Vec8<__nv_bfloat16>::load(const __nv_bfloat16* p) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void Vec8<__nv_bfloat16>::store(__nv_bfloat16* p) const {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// tanh-form GELU of the reference (layers/kernels/activation.cpp:32-55).
__device__ __forceinline__ float gelu_tanh(float x) {
  return x * 0.5f * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

// Dispatch a templated launcher on the floating dtypes.
#define TTB_DISPATCH_FLOAT(ctx, dtype, T, ...)                                         \
  switch (dtype) {                                                                     \
    case TTB_F32: { using T = float; __VA_ARGS__; break; }                             \
    case TTB_F16: { using T = __half; __VA_ARGS__; break; }                            \
    case TTB_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }                    \
    default: return ::ttb::fail(ctx, TTB_ERR_UNSUPPORTED, "unsupported dtype %d", (int)(dtype)); \
  }

}  // namespace ttb
