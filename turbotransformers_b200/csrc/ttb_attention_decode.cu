// Decoder step over a key/value cache: the new tokens' keys and values are appended in place and the new queries attend
// everything cached so far. Replaces the reference's per-step Concat of the whole cache plus its padded attention sequence
// (multi_headed_attention.cpp:207-231 and 320-354) for `layer_cache` self-attention.
//
// Caches are paged: [pages, B, 16, H] (H = heads * 64), page p holding tokens 16p .. 16p+15 of every sequence. Appending writes
// in place, growth adds pages at the end, and the 16 tokens of a sequence inside a page are 24 KB of contiguous memory that the
// CTAs of its heads read together (a time-major [T, B, H] layout measured 47 % of the copy bandwidth: every 128-byte row in its
// own DRAM page). The kernel is bound by reading K and V once: B * T * H * 4 bytes per call.
//   grid (heads, B), 128 threads. Eight lanes share a key (16 bytes of it each), so a warp covers four keys per load and
//   the four warps sixteen; scores are reduced over the eight lanes with three shuffles, softmax is kept online per lane
//   group and the sixteen partial (max, sum, output) states are merged through shared memory at the end.
#include "ttb_common.cuh"

using namespace ttb;

namespace {

constexpr int D = 64;
constexpr int kThreads = 128;
constexpr int kGroups = kThreads / 8;  // key groups per CTA == tokens per cache page
constexpr int kPage = 16;
static_assert(kGroups == kPage, "lane group g reads row g of every page");

// element offset of token j of sequence b inside a paged cache
__device__ __forceinline__ long long cache_row(int j, int b, int B, int H) {
  return (((long long)(j >> 4) * B + b) * kPage + (j & 15)) * H;
}
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8], const __half*) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8], const __nv_bfloat16*) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
kv_append_kernel(const T* __restrict__ qkv, int B, int n_new, int H, T* __restrict__ kc, T* __restrict__ vc, int past_len) {
  // one 16-byte chunk of one K row and of one V row per thread
  const int chunks = H / 8;
  const long long total = (long long)B * n_new * chunks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks);
    const long long row = i / chunks;  // b * n_new + t
    const int b = (int)(row / n_new), t = (int)(row % n_new);
    const T* src = qkv + row * 3ll * H + H + c * 8;
    const long long dst = cache_row(past_len + t, b, B, H) + c * 8;
    *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(src + H);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 5)
attention_decode_kernel(const T* __restrict__ qkv, int B, int n_new, int heads, T* __restrict__ kc, T* __restrict__ vc, int past_len,
                        float scale, T* __restrict__ out) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int H = heads * D;
  const int tid = threadIdx.x, lane = tid & 31, sub = lane & 7, group = tid >> 3;
  __shared__ float s_m[kGroups], s_l[kGroups];
  __shared__ float s_acc[kGroups][D];

  // append this head's new keys and values: 16-byte chunks, 8 per row
  for (int i = tid; i < n_new * 16; i += kThreads) {
    const int t = i >> 4, which = (i >> 3) & 1, c = i & 7;
    const T* src = qkv + ((long long)(b * n_new + t)) * 3 * H + (1 + which) * H + h * D + c * 8;
    T* dst = (which ? vc : kc) + cache_row(past_len + t, b, B, H) + h * D + c * 8;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
  __syncthreads();  // this CTA reads back what it has just written (same block: ordered by the barrier)

  // lane group g reads row g of page after page: token j = 16 * page + g
  const long long page_stride = (long long)B * kPage * H;
  const T* kbase = kc + ((long long)b * kPage + group) * H + h * D + sub * 8;
  const T* vbase = vc + ((long long)b * kPage + group) * H + h * D + sub * 8;
  for (int t = 0; t < n_new; ++t) {
    // this lane's eight query elements, scale and log2(e) folded in
    float q[8];
    {
      Vec8<T> qv;
      qv.load(qkv + ((long long)(b * n_new + t)) * 3 * H + h * D + sub * 8);
#pragma unroll
      for (int e = 0; e < 8; ++e) q[e] = qv.v[e] * scale * kLog2e;
    }
    const int n_keys = past_len + t + 1;  // query t sees the cache and the new tokens up to itself
    float m = -INFINITY, l = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // The trip count is the same for every thread of the CTA (the shuffles below are full-warp): a lane group whose key
    // index runs past the end only skips the loads and the update. Four keys per lane group per round, and the next
    // round's 16-byte loads are issued before the current round is consumed.
    auto load_round = [&](int base, uint4 (&kr)[4], uint4 (&vr)[4]) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = base + group + u * kGroups;
        if (j < n_keys) {
          kr[u] = *reinterpret_cast<const uint4*>(kbase + (j >> 4) * page_stride);
          vr[u] = *reinterpret_cast<const uint4*>(vbase + (j >> 4) * page_stride);
        }
      }
    };
    uint4 kr[4], vr[4];
    load_round(0, kr, vr);
    for (int base = 0; base < n_keys; base += 4 * kGroups) {
      uint4 kn[4], vn[4];
      if (base + 4 * kGroups < n_keys) load_round(base + 4 * kGroups, kn, vn);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool live = base + group + u * kGroups < n_keys;
        float s = 0.f;
        if (live) {
          float kf[8];
          unpack8(kr[u], kf, static_cast<const T*>(nullptr));
#pragma unroll
          for (int e = 0; e < 8; ++e) s = fmaf(q[e], kf[e], s);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (live) {
          float vf[8];
          unpack8(vr[u], vf, static_cast<const T*>(nullptr));
          const float m_new = fmaxf(m, s);
          const float corr = ex2f(m - m_new), p = ex2f(s - m_new);
          l = l * corr + p;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(p, vf[e], acc[e] * corr);
          m = m_new;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        kr[u] = kn[u];
        vr[u] = vn[u];
      }
    }
    // merge the lane groups' partial states
    if (sub == 0) {
      s_m[group] = m;
      s_l[group] = l;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s_acc[group][sub * 8 + e] = acc[e];
    __syncthreads();
    if (tid < D) {
      float M = -INFINITY;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) M = fmaxf(M, s_m[g]);
      float L = 0.f, o = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const float w = ex2f(s_m[g] - M);  // 0 for a group that saw no key
        L = fmaf(s_l[g], w, L);
        o = fmaf(s_acc[g][tid], w, o);
      }
      out[((long long)(b * n_new + t)) * H + h * D + tid] = from_f<T>(o / L);
    }
    __syncthreads();
  }
}

int check_decode(ttb_ctx* ctx, const char* what, int dtype, const void* qkv, int64_t B, int64_t n_new, int64_t heads, int64_t d,
                 const void* kc, const void* vc, int64_t past_len) {
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "%s: dtype must be F16 or BF16", what);
  TTB_REQUIRE(ctx, d == D, "%s: head size must be 64", what);
  TTB_REQUIRE(ctx, B > 0 && n_new > 0 && heads > 0 && past_len >= 0, "%s: bad shape", what);
  TTB_REQUIRE(ctx, B <= 65535 && (past_len + n_new) * B * heads * d < (1ll << 40), "%s: shape too large", what);
  TTB_REQUIRE(ctx, qkv && kc && vc, "%s: null pointer", what);
  TTB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc)) & 15) == 0,
              "%s: buffers must be 16-byte aligned", what);
  return TTB_OK;
}

}  // namespace

extern "C" int ttb_kv_cache_append(ttb_ctx* ctx, int dtype, const void* qkv, int64_t B, int64_t n_new, int64_t heads, int64_t d, void* k_cache,
                                   void* v_cache, int64_t past_len) {
  if (!ctx) return TTB_ERR_INVALID;
  int s = check_decode(ctx, "kv_cache_append", dtype, qkv, B, n_new, heads, d, k_cache, v_cache, past_len);
  if (s) return s;
  DeviceGuard g(ctx->device);
  const int H = (int)(heads * d);
  const long long total = B * n_new * (H / 8);
  const int grid = (int)std::min<long long>((total + kThreads - 1) / kThreads, (long long)ctx->sm_count * 16);
  if (dtype == TTB_F16)
    kv_append_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>((const __half*)qkv, (int)B, (int)n_new, H, (__half*)k_cache, (__half*)v_cache,
                                                                  (int)past_len);
  else
    kv_append_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16*)qkv, (int)B, (int)n_new, H, (__nv_bfloat16*)k_cache,
                                                                         (__nv_bfloat16*)v_cache, (int)past_len);
  return launched(ctx, "kv_cache_append");
}

extern "C" int ttb_attention_decode(ttb_ctx* ctx, int dtype, const void* qkv, int64_t B, int64_t n_new, int64_t heads, int64_t d, void* k_cache,
                                    void* v_cache, int64_t past_len, float scale, void* out) {
  if (!ctx) return TTB_ERR_INVALID;
  int s = check_decode(ctx, "attention_decode", dtype, qkv, B, n_new, heads, d, k_cache, v_cache, past_len);
  if (s) return s;
  TTB_REQUIRE(ctx, out, "attention_decode: null output");
  TTB_REQUIRE(ctx, n_new <= 64, "attention_decode: at most 64 new tokens per call (use ttb_attention_fwd + ttb_kv_cache_append for a prompt)");
  DeviceGuard g(ctx->device);
  dim3 grid((unsigned)heads, (unsigned)B);
  if (dtype == TTB_F16)
    attention_decode_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>((const __half*)qkv, (int)B, (int)n_new, (int)heads, (__half*)k_cache,
                                                                         (__half*)v_cache, (int)past_len, scale, (__half*)out);
  else
    attention_decode_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16*)qkv, (int)B, (int)n_new, (int)heads,
                                                                                (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (int)past_len,
                                                                                scale, (__nv_bfloat16*)out);
  return launched(ctx, "attention_decode");
}
