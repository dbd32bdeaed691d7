// int8 Linear with dynamic activation quantisation for callers that cannot allocate device memory.
//
// Some hosts hand this library nothing but input and output buffers: a serving loop that has already given all
// device memory to its own arena, code running inside a region where the CUDA allocator must not be called (its own
// bookkeeping is not re-entrant there), or an embedding runtime whose FFI has no way to own device buffers. The
// regular int8 path needs two scratch buffers between its kernels (the quantised activations and their per-row
// scales) which the caller normally provides. Here they live in a fixed array inside the library image instead.
#include <mutex>

#include "ttb_common.cuh"

using namespace ttb;

namespace {

constexpr size_t kMaxActivationBytes = size_t(8) << 20;  // int8 activations: M*K <= 8 Mi
constexpr size_t kMaxRows = size_t(1) << 16;             // per-row scales: M <= 65 536
constexpr size_t kScratchBytes = kMaxActivationBytes + kMaxRows * sizeof(float);

// Held by every GPU that loads the library, from load until process exit (8.25 MiB). In host code this name is only a
// handle for the runtime: the device address is asked for once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

std::mutex g_mu;
unsigned char* g_scratch_ptr[64] = {};

// The scratch array's address on `ctx`'s device (looked up on the first call for that device).
int scratch_for(ttb_ctx* ctx, unsigned char** out) {
  const int dev = ctx->device;
  if (dev < 0 || dev >= 64) return fail(ctx, TTB_ERR_INVALID, "linear_int8_dynamic_noalloc: device id %d out of range", dev);
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_scratch_ptr[dev]) {
    DeviceGuard guard(dev);  // the symbol has one instance per device: resolve it with that device current
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(ctx, TTB_ERR_CUDA, "linear_int8_dynamic_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return TTB_OK;
}

}  // namespace

extern "C" int ttb_linear_int8_dynamic_noalloc(ttb_ctx* ctx, int dtype, const void* x, const int8_t* Wq, const float* w_scale,
                                               const void* bias, const void* residual, int64_t ldr, int64_t M, int64_t N,
                                               int64_t K, int epilogue, void* out, int64_t ldo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M >= 0 && N > 0 && K > 0, "linear_int8_dynamic_noalloc: bad shape");
  TTB_REQUIRE(ctx, (uint64_t)M <= kMaxRows && (uint64_t)M * (uint64_t)K <= kMaxActivationBytes,
              "linear_int8_dynamic_noalloc: M=%lld K=%lld exceeds the built-in scratch (M <= %zu rows and M*K <= %zu); "
              "use ttb_quantize_rows_int8 + ttb_linear_int8 with caller-provided buffers for larger problems",
              (long long)M, (long long)K, kMaxRows, kMaxActivationBytes);
  // Everything the two kernels below would reject is rejected here, so that a refused call has launched nothing and
  // has not touched the shared scratch.
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "linear_int8_dynamic_noalloc: dtype must be F16 or BF16");
  TTB_REQUIRE(ctx, epilogue >= TTB_EPI_NONE && epilogue <= TTB_EPI_BIAS_TANH, "linear_int8_dynamic_noalloc: unknown epilogue %d", epilogue);
  TTB_REQUIRE(ctx, K % 16 == 0, "linear_int8_dynamic_noalloc: K=%lld must be a multiple of 16", (long long)K);
  TTB_REQUIRE(ctx, ldo >= N, "linear_int8_dynamic_noalloc: ldo < N");
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, x && Wq && w_scale && out, "linear_int8_dynamic_noalloc: null pointer");
  TTB_REQUIRE(ctx, epilogue == TTB_EPI_NONE || bias, "linear_int8_dynamic_noalloc: epilogue %d needs a bias", epilogue);
  TTB_REQUIRE(ctx, epilogue != TTB_EPI_BIAS_RESIDUAL || residual, "linear_int8_dynamic_noalloc: the residual epilogue needs a residual");
  TTB_REQUIRE(ctx, reinterpret_cast<uintptr_t>(Wq) % 16 == 0, "linear_int8_dynamic_noalloc: the weights must be 16-byte aligned");
  unsigned char* scratch = nullptr;
  int s = scratch_for(ctx, &scratch);
  if (s != TTB_OK) return s;
  int8_t* xq = reinterpret_cast<int8_t*>(scratch);
  float* row_scale = reinterpret_cast<float*>(scratch + kMaxActivationBytes);
  // Both kernels overwrite every scratch element they later read (M*K activations, M scales), so nothing from an
  // earlier call has to be cleared.
  s = ttb_quantize_rows_int8(ctx, dtype, x, M, K, xq, row_scale);
  if (s != TTB_OK) return s;
  return ttb_linear_int8(ctx, dtype, xq, row_scale, Wq, w_scale, bias, residual, ldr, M, N, K, epilogue, out, ldo);
}
