// Decoder step over a key/value cache: the new tokens' keys and values are appended in place and the new queries attend
// everything cached so far. Replaces the reference's per-step Concat of the whole cache plus its padded attention sequence
// (multi_headed_attention.cpp:207-231 and 320-354) for `layer_cache` self-attention.
//
// Caches are paged: [pages, B, 16, H] (H = heads * 64), page p holding tokens 16p .. 16p+15 of every sequence. Appending writes
// in place, growth adds pages at the end, and the 16 tokens of a sequence inside a page are 24 KB of contiguous memory that the
// CTAs of its heads read together (a time-major [T, B, H] layout measured 47 % of the copy bandwidth: every 128-byte row in its
// own DRAM page). The kernel is bound by reading K and V once: B * T * H * 4 bytes per call.
//   grid (heads, B, splits), 128 threads. Eight lanes share a key (16 bytes of it each), so a warp covers four keys per load
//   and the four warps sixteen (one cache page); scores are reduced over the eight lanes with three shuffles, softmax is kept
//   online per lane group and the sixteen partial (max, sum, output) states are merged through shared memory at the end.
//   With few (sequence, head) pairs the pages are split over several CTAs and a second kernel merges their partial states.
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

// Partial result of one split of one (sequence, head, new token): running maximum (log2 units), sum and 64 output sums.
constexpr int kPartial = D + 2;

template <typename T>
__global__ void __launch_bounds__(kThreads, 5)
attention_decode_kernel(const T* __restrict__ qkv, int B, int n_new, int heads, T* __restrict__ kc, T* __restrict__ vc, int past_len,
                        float scale, T* __restrict__ out, float* __restrict__ partial, int splits) {
  const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int H = heads * D;
  const int tid = threadIdx.x, lane = tid & 31, sub = lane & 7, group = tid >> 3;
  __shared__ float s_m[kGroups], s_l[kGroups];
  __shared__ float s_acc[kGroups][D];

  // append this head's new keys and values: 16-byte chunks, 8 per row (every split writes the same bytes: the splits of a
  // (sequence, head) are different CTAs and each reads the new rows back after its own barrier)
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
    // this split's pages: a contiguous range, the same for every thread of the CTA (the shuffles below are full-warp)
    const int n_pages = (n_keys + kPage - 1) / kPage;
    const int per = (n_pages + splits - 1) / splits;
    const int p_begin = split * per, p_end = min(n_pages, p_begin + per);
    // Two independent running states per lane (even / odd pages), so consecutive keys do not wait on each other's
    // maximum / rescale chain; four pages per round are in flight per lane group.
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, acc[2][8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[0][e] = acc[1][e] = 0.f;
    for (int pg = p_begin; pg < p_end; pg += 4) {
      uint4 kr[4], vr[4];
      bool live[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        live[u] = (pg + u < p_end) && ((pg + u) * kPage + group < n_keys);
        if (live[u]) {
          kr[u] = *reinterpret_cast<const uint4*>(kbase + (pg + u) * page_stride);
          vr[u] = *reinterpret_cast<const uint4*>(vbase + (pg + u) * page_stride);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float s = 0.f;
        if (live[u]) {
          float kf[8];
          unpack8(kr[u], kf, static_cast<const T*>(nullptr));
#pragma unroll
          for (int e = 0; e < 8; ++e) s = fmaf(q[e], kf[e], s);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (live[u]) {
          float vf[8];
          unpack8(vr[u], vf, static_cast<const T*>(nullptr));
          const int w = u & 1;
          const float m_new = fmaxf(m[w], s);
          const float corr = ex2f(m[w] - m_new), p = ex2f(s - m_new);
          l[w] = l[w] * corr + p;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[w][e] = fmaf(p, vf[e], acc[w][e] * corr);
          m[w] = m_new;
        }
      }
    }
    // fold the two states of this lane, then merge the lane groups' partial states
    {
      const float M = fmaxf(m[0], m[1]);
      const float w0 = (m[0] == -INFINITY) ? 0.f : ex2f(m[0] - M), w1 = (m[1] == -INFINITY) ? 0.f : ex2f(m[1] - M);
      l[0] = l[0] * w0 + l[1] * w1;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[0][e] = acc[0][e] * w0 + acc[1][e] * w1;
      m[0] = M;
    }
    if (sub == 0) {
      s_m[group] = m[0];
      s_l[group] = l[0];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s_acc[group][sub * 8 + e] = acc[0][e];
    __syncthreads();
    if (tid < D) {
      float M = -INFINITY;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) M = fmaxf(M, s_m[g]);
      float L = 0.f, o = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const float w = (s_m[g] == -INFINITY) ? 0.f : ex2f(s_m[g] - M);  // a group that saw no key
        L = fmaf(s_l[g], w, L);
        o = fmaf(s_acc[g][tid], w, o);
      }
      if (splits == 1) {
        out[((long long)(b * n_new + t)) * H + h * D + tid] = from_f<T>(o / L);
      } else {
        float* dst = partial + ((((long long)(b * n_new + t)) * heads + h) * splits + split) * kPartial;
        dst[2 + tid] = o;
        if (tid == 0) {
          dst[0] = M;
          dst[1] = L;
        }
      }
    }
    __syncthreads();
  }
}

// out = merge of the splits' partial states, one warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(128)
decode_merge_kernel(const float* __restrict__ partial, int rows_heads, int splits, int heads, T* __restrict__ out) {
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= rows_heads) return;
  const float* p = partial + (long long)item * splits * kPartial;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, p[s * kPartial]);
  float L = 0.f, o0 = 0.f, o1 = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = p[s * kPartial];
    const float w = (ms == -INFINITY) ? 0.f : ex2f(ms - M);  // a split that had no pages
    L = fmaf(p[s * kPartial + 1], w, L);
    o0 = fmaf(p[s * kPartial + 2 + lane], w, o0);
    o1 = fmaf(p[s * kPartial + 2 + 32 + lane], w, o1);
  }
  const int row = item / heads, h = item % heads;
  T* dst = out + (long long)row * heads * D + h * D;
  dst[lane] = from_f<T>(o0 / L);
  dst[32 + lane] = from_f<T>(o1 / L);
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
  // A (sequence, head) is one CTA's serial walk over its keys; with few of them the keys are split over several CTAs (each
  // at least 8 pages = 128 keys) until there are about eight CTAs per SM, and a second kernel merges the partial states.
  const int64_t ctas = heads * B, pages = (past_len + n_new + kPage - 1) / kPage;
  int splits = (int)std::min<int64_t>(std::min<int64_t>((8ll * ctx->sm_count + ctas - 1) / ctas, pages / 8), 16);
  if (splits < 1) splits = 1;
  float* partial = nullptr;
  if (splits > 1) {
    void* p = nullptr;
    s = ttb_alloc(ctx, (size_t)(B * n_new * heads * splits * kPartial) * sizeof(float), "attention_decode/partials", &p);
    if (s) return s;
    partial = static_cast<float*>(p);
  }
  dim3 grid((unsigned)heads, (unsigned)B, (unsigned)splits);
  const int items = (int)(B * n_new * heads);
  if (dtype == TTB_F16) {
    attention_decode_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>((const __half*)qkv, (int)B, (int)n_new, (int)heads, (__half*)k_cache,
                                                                         (__half*)v_cache, (int)past_len, scale, (__half*)out, partial, splits);
    if (splits > 1) decode_merge_kernel<__half><<<(items + 3) / 4, 128, 0, ctx->stream>>>(partial, items, splits, (int)heads, (__half*)out);
  } else {
    attention_decode_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16*)qkv, (int)B, (int)n_new, (int)heads,
                                                                                (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (int)past_len,
                                                                                scale, (__nv_bfloat16*)out, partial, splits);
    if (splits > 1)
      decode_merge_kernel<__nv_bfloat16><<<(items + 3) / 4, 128, 0, ctx->stream>>>(partial, items, splits, (int)heads, (__nv_bfloat16*)out);
  }
  s = launched(ctx, "attention_decode");
  if (partial) {
    const int f = ttb_free(ctx, partial, "attention_decode/partials");  // stream-ordered: released after the merge has run
    if (!s) s = f;
  }
  return s;
}
