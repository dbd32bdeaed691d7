// Self-attention over packed, variable-length token batches: softmax(Q K^T * scale + mask) V per
// (sequence, head), computed tile by tile with an online softmax so the score matrix never reaches HBM.
//
// Input is the QKV projection as the GEMM wrote it, [tokens, 3*heads*64] with columns q|k|v, so no
// split/transpose kernel runs before and no un-transpose after: the output is written as [tokens, heads*64].
// Sequences are addressed through cu_seqlens (prefix sums of lengths); nothing is padded.
//
// CTA = 4 warps = 64 query rows of one (sequence, head); keys/values stream through a double-buffered
// cp.async ring of 64-row tiles (16-byte chunks XOR-swizzled so ldmatrix is conflict-free); the two
// contractions run on mma.sync m16n8k16 with fp32 accumulation, softmax statistics in fp32.
#include "ttb_common.cuh"

using namespace ttb;

namespace {

constexpr int D = 64;        // head size
constexpr int QT = 64;       // query rows per CTA
constexpr int KT = 64;       // key rows per tile
constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of 16-byte chunk `c` (0..7) of row `r` inside a [rows x 128 B] tile
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// 2^x by the special-function unit (2 ulp); 2^-inf = +0.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnParams {
  const void* qkv;
  void* out;
  const int32_t* cu;
  const float* mask;
  long long mask_bs, mask_rs;
  int heads, causal;
  float scale;
};

// Copies rows [row0, row0+64) of one head's q, k or v slice into a swizzled tile; rows >= len are zero-filled.
template <typename T>
__device__ __forceinline__ void load_tile(uint32_t tile, const T* base, long long ld, int row0, int len, int tid) {
#pragma unroll
  for (int i = 0; i < (QT * 8) / (kWarps * 32); ++i) {
    const int idx = tid + i * kWarps * 32;
    const int r = idx >> 3, c = idx & 7;
    const bool valid = row0 + r < len;
    const T* src = base + (long long)(valid ? row0 + r : 0) * ld + c * 8;
    cp_async16(tile + swz(r, c), src, valid);
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_fwd_kernel(const AttnParams p) {
  __shared__ __align__(128) uint8_t sQ[QT * 128];
  __shared__ __align__(128) uint8_t sK[2][KT * 128];
  __shared__ __align__(128) uint8_t sV[2][KT * 128];

  pdl_trigger();
  pdl_wait();  // before the first global read and before any CTA can leave
  const int b = blockIdx.z, h = blockIdx.y;
  const int tok0 = p.cu[b];
  const int len = p.cu[b + 1] - tok0;
  const int q0 = blockIdx.x * QT;
  if (q0 >= len) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.heads * D;
  const long long ld = 3ll * H;
  const T* qkv = static_cast<const T*>(p.qkv);
  const T* qb = qkv + (long long)tok0 * ld + h * D;
  const T* kb = qb + H;
  const T* vb = qb + 2 * H;

  const uint32_t sq = smem_u32(sQ);
  const uint32_t sk[2] = {smem_u32(sK[0]), smem_u32(sK[1])};
  const uint32_t sv[2] = {smem_u32(sV[0]), smem_u32(sV[1])};

  int kv_end = len;
  if (p.causal && q0 + QT < kv_end) kv_end = q0 + QT;
  const int n_tiles = (kv_end + KT - 1) / KT;

  load_tile<T>(sq, qb, ld, q0, len, tid);
  load_tile<T>(sk[0], kb, ld, 0, len, tid);
  load_tile<T>(sv[0], vb, ld, 0, len, tid);
  cp_async_commit();

  uint32_t qf[4][4];
  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int g = lane >> 2, t4 = lane & 3;
  const int qrow[2] = {q0 + warp * 16 + g, q0 + warp * 16 + g + 8};
  const float sc = p.scale * kLog2e;
  const float* mrow[2] = {nullptr, nullptr};
  if (p.mask) {
    mrow[0] = p.mask + (long long)b * p.mask_bs + (long long)qrow[0] * p.mask_rs;
    mrow[1] = p.mask + (long long)b * p.mask_bs + (long long)qrow[1] * p.mask_rs;
  }

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) {
      load_tile<T>(sk[buf ^ 1], kb, ld, (t + 1) * KT, len, tid);
      load_tile<T>(sv[buf ^ 1], vb, ld, (t + 1) * KT, len, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    if (t == 0) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldsm_x4(qf[kk], sq + swz(r, kk * 2 + (lane >> 4)));
      }
    }

    // ---- S = Q K^T for 16 query rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t kf[4];
        const int m = lane >> 3;
        ldsm_x4(kf, sk[buf] + swz((j + (m >> 1)) * 8 + (lane & 7), kk * 2 + (m & 1)));
        mma16816<T>(s[j], qf[kk], kf[0], kf[1]);
        mma16816<T>(s[j + 1], qf[kk], kf[2], kf[3]);
      }
    }

    // ---- scale, mask, online softmax (rows g and g+8 of this warp's 16)
    const int k0 = t * KT;
    // Per-element masking only where a tile needs it (warp-uniform): a mask tensor, keys past the end of the
    // sequence, or the causal diagonal. Interior tiles keep the raw scores and fold the scale into the exp2 FMA.
    // A mask with one row of keys per sequence (the encoder's padding mask) is zero over most tiles: the warp looks at the
    // tile's entries once and treats the tile as unmasked when none of them is set.
    bool mask_set = p.mask != nullptr;
    if (p.mask && p.mask_rs == 0) {
      const float* mr = p.mask + (long long)b * p.mask_bs + k0;
      bool mine = false;
#pragma unroll
      for (int u = 0; u < KT; u += 32) mine = mine || (k0 + u + lane < len && mr[u + lane] != 0.f);
      mask_set = __any_sync(0xffffffffu, mine);
    }
    const bool edge = mask_set || (k0 + KT > len) || (p.causal && k0 + KT - 1 > q0 + warp * 16);
    float sce = sc;
    if (edge) {
      sce = 1.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int key = k0 + j * 8 + t4 * 2 + (e & 1);
          float v = s[j][e] * sc;
          const bool dead = key >= len || (p.causal && key > qrow[r]);
          if (mask_set && !dead && qrow[r] < len) v += mrow[r][key] * kLog2e;
          s[j][e] = dead ? -INFINITY : v;
        }
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r] * sce);
      // m_new is finite from the first tile on (key 0 is never dead); guard the degenerate all-dead row anyway
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      corr[r] = ex2(m_run[r] - m_use);
      m_run[r] = m_new;
      mx[r] = m_use;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float pv = ex2(fmaf(s[j][e], sce, -mx[r]));
        s[j][e] = pv;
        rs[r] += pv;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * corr[r] + rs[r];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }

    // ---- O += P V
#pragma unroll
    for (int kt = 0; kt < 4; ++kt) {
      uint32_t pf[4];
      pf[0] = pack2<T>(s[2 * kt][0], s[2 * kt][1]);
      pf[1] = pack2<T>(s[2 * kt][2], s[2 * kt][3]);
      pf[2] = pack2<T>(s[2 * kt + 1][0], s[2 * kt + 1][1]);
      pf[3] = pack2<T>(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
      for (int jd = 0; jd < 8; jd += 2) {
        uint32_t vf[4];
        const int m = lane >> 3;
        ldsm_x4_trans(vf, sv[buf] + swz(kt * 16 + (m & 1) * 8 + (lane & 7), jd + (m >> 1)));
        mma16816<T>(o[jd], pf, vf[0], vf[1]);
        mma16816<T>(o[jd + 1], pf, vf[2], vf[3]);
      }
    }
    __syncthreads();  // everyone is done with buf before the next iteration's prefetch overwrites it
  }

  // ---- normalise, stage through this warp's rows of the Q tile, write 16-byte rows
  const float inv[2] = {1.0f / l_run[0], 1.0f / l_run[1]};
#pragma unroll
  for (int jd = 0; jd < 8; ++jd) {
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    // chunk jd holds d = jd*8 .. jd*8+7; this thread owns elements t4*2, t4*2+1 of it
    *reinterpret_cast<uint32_t*>(sQ + swz(r0, jd) + t4 * 4) = pack2<T>(o[jd][0] * inv[0], o[jd][1] * inv[0]);
    *reinterpret_cast<uint32_t*>(sQ + swz(r1, jd) + t4 * 4) = pack2<T>(o[jd][2] * inv[1], o[jd][3] * inv[1]);
  }
  __syncwarp();
  T* ob = static_cast<T*>(p.out) + (long long)tok0 * H + h * D;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp * 16 + i * 4 + (lane >> 3), c = lane & 7;
    if (q0 + r < len) {
      const uint4 v = *reinterpret_cast<const uint4*>(sQ + swz(r, c));
      *reinterpret_cast<uint4*>(ob + (long long)(q0 + r) * H + c * 8) = v;
    }
  }
}

}  // namespace

namespace ttb {
int attention_tc_mode();
int attention_tc_launch(ttb_ctx* ctx, int dtype, const void* qkv, int64_t tokens, const int32_t* cu, int64_t B, int64_t max_seqlen,
                        int64_t heads, const float* mask, int64_t mask_batch_stride, int causal, float scale, void* out);
}  // namespace ttb

extern "C" int ttb_attention_fwd(ttb_ctx* ctx, int dtype, const void* qkv, int64_t total_tokens, const int32_t* cu_seqlens,
                                 int64_t B, int64_t max_seqlen, int64_t heads, int64_t d, const float* mask,
                                 int64_t mask_batch_stride, int64_t mask_row_stride, int causal, float scale,
                                 void* out) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "attention_fwd: dtype must be F16 or BF16");
  TTB_REQUIRE(ctx, d == D, "attention_fwd: head size must be 64 (got %lld)", (long long)d);
  TTB_REQUIRE(ctx, B >= 0 && max_seqlen >= 0 && heads > 0 && heads <= 65535 && B <= 65535, "attention_fwd: bad shape");
  if (B == 0 || max_seqlen == 0) return TTB_OK;
  TTB_REQUIRE(ctx, qkv && cu_seqlens && out, "attention_fwd: null pointer");
  TTB_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out)) % 16 == 0,
              "attention_fwd: qkv and out must be 16-byte aligned");
  TTB_REQUIRE(ctx, total_tokens >= 0, "attention_fwd: negative token count");
  DeviceGuard g(ctx->device);
  // The persistent tensor-memory kernel wins once its 128 x 128 tiles are mostly full and there is enough work to fill its
  // pipeline; short sequences (one key tile per item, query tiles half empty) and small batches finish sooner on the many
  // small CTAs of the mma.sync kernel, which also serves masks with a row per query (a mask with one row of keys per
  // sequence, the encoder's padding mask, is an operand of the tensor-memory kernel). Measured on B200, graph replay, us,
  // tensor-memory / mma.sync: 4 x 512 16.0 / 20.7, 3 x 1024 24.7 / 38.9, 2 x 512 14.8 / 12.5, 16 x 256 18.4 / 17.7,
  // 64 x 128 20.3 / 18.4, 128 x 64 36.7 / 13.9; the ragged benchmark batch (64 sequences of 8..512) 80 / 96.
  // With a padding mask the tensor-memory kernel is ahead much earlier (16 x 256 20.0 / 30.5, 8 x 512 28.6 / 56.1).
  const bool enough_work = mask ? total_tokens * max_seqlen >= (1ll << 19) : (max_seqlen >= 384 && total_tokens * max_seqlen >= (1ll << 20));
  const int tc_mode = attention_tc_mode();
  if ((!mask || mask_row_stride == 0) && total_tokens > 0 && (tc_mode == 2 || (tc_mode == 1 && enough_work))) {
    const int s = attention_tc_launch(ctx, dtype, qkv, total_tokens, cu_seqlens, B, max_seqlen, heads, mask, mask_batch_stride, causal, scale, out);
    if (s != TTB_ERR_UNSUPPORTED) return s;
  }
  AttnParams p{qkv, out, cu_seqlens, mask, mask_batch_stride, mask_row_stride, (int)heads, causal ? 1 : 0, scale};
  dim3 grid((unsigned)((max_seqlen + QT - 1) / QT), (unsigned)heads, (unsigned)B);
  if (dtype == TTB_F16) launch_pdl(attention_fwd_kernel<__half>, grid, dim3(kWarps * 32), 0, ctx->stream, p);
  else launch_pdl(attention_fwd_kernel<__nv_bfloat16>, grid, dim3(kWarps * 32), 0, ctx->stream, p);
  return launched(ctx, "attention_fwd");
}
