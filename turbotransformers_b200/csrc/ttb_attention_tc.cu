// Self-attention over packed variable-length batches on the 5th-generation tensor cores.
//
// One CTA = 128 query rows of one (sequence, head). Keys/values stream in 128-row tiles.
//   warp 0     : TMA loader   - Q once, then K_j and V_j tiles (128-byte-swizzled, straight out of the [T, 3H] QKV
//                matrix: a tile is a [128 rows x 64 columns] box at column offset part*H + head*64) into a 2-slot ring
//   warp 1     : MMA issuer   - S = Q K_j^T (128x128x64, accumulator in TMEM), then O_j = P_j V_j (128x64x128) with
//                P_j read from shared memory and V_j used in place as an MN-major operand (no transpose anywhere)
//   warps 2..5 : softmax      - one query row per thread: tcgen05.ld the scores, running max / sum in fp32, exp2 with the
//                scale folded in, P_j written to shared memory as the next MMA's K-major A operand. O accumulates in
//                TMEM across tiles and is rescaled there only when the running maximum has grown by more than 2^8
// TMEM: S (128 columns) + O (64 columns) inside a 256-column allocation, so two CTAs fit on an SM and one CTA's
// softmax overlaps the other's MMAs. Every wait is bounded; on expiry the CTA raises a flag, frees its TMEM and the host
// sees TTB_ERR_DEVICE_WAIT.
#include <cstdlib>
#include <type_traits>

#include "ttb_common.cuh"
#include "ttb_sm100.cuh"

using namespace ttb;
using namespace ttb::sm100;

namespace {

constexpr int QT = 128, KT = 128, D = 64;
constexpr int kThreads = 192;
constexpr int TILE_BYTES = 128 * 128;          // a [128 rows x 128 B] tile
constexpr int SMEM_Q = 0, SMEM_K = TILE_BYTES, SMEM_V = 3 * TILE_BYTES, SMEM_P = 5 * TILE_BYTES;  // K,V: 2 slots; P: 2 atoms
constexpr int SMEM_BARS = 7 * TILE_BYTES;
constexpr int SMEM_BYTES = 7 * TILE_BYTES + 128;  // two CTAs per SM: 2 x (112.1 KB + 1 KB reserved) <= 228 KB
constexpr uint32_t TMEM_COLS = 256;
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  void* out;
  const int32_t* cu;
  int heads, causal;
  float scale;
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap tm, const Params p) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int tok0 = p.cu[b];
  const int len = p.cu[b + 1] - tok0;
  const int q0 = blockIdx.x * QT;
  if (q0 >= len) return;  // whole CTA, before any barrier or TMEM use

  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_S = idesc_f16(FMT, 128, KT, 0);   // Q (K-major) x K^T (K-major)
  constexpr uint32_t IDESC_O = idesc_f16(FMT, 128, D, 1);    // P (K-major) x V (MN-major)

  extern __shared__ __align__(1024) uint8_t smem[];  // the swizzled tiles need 1024-byte alignment
  const uint32_t base = smem_u32(smem);
  if (base & 1023u) {  // cannot happen with the alignment above; refuse rather than compute garbage
    if (threadIdx.x == 0) atomicExch(p.status, (int)TTB_ERR_DEVICE_WAIT);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BARS);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0, s_full = bar0 + 8, s_empty = bar0 + 16, p_full = bar0 + 24;
  auto kv_full = [&](int s) { return bar0 + 32 + 8u * s; };
  auto kv_empty = [&](int s) { return bar0 + 48 + 8u * s; };
  auto o_full = [&](int s) { return bar0 + 64 + 8u * s; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = p.heads * D;
  int kv_end = len;
  if (p.causal && q0 + QT < kv_end) kv_end = q0 + QT;
  const int n_tiles = (kv_end + KT - 1) / KT;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(s_empty, 4);
    mbar_init(p_full, 4);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
      mbar_init(o_full(s), 1);
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s = tmem, tmem_o0 = tmem + 128;

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_2d(base + SMEM_Q, &tm, q_full, h * D, tok0 + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(kv_empty(s), (((uint32_t)j >> 1) & 1u) ^ 1u, abort_flag)) break;
        mbar_expect_tx(kv_full(s), 2 * TILE_BYTES);
        tma_load_2d(base + SMEM_K + s * TILE_BYTES, &tm, kv_full(s), H + h * D, tok0 + j * KT);
        tma_load_2d(base + SMEM_V + s * TILE_BYTES, &tm, kv_full(s), 2 * H + h * D, tok0 + j * KT);
      }
      if (*abort_flag) {  // let copies in flight land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag);
      const uint32_t q_lo = desc_lo(base + SMEM_Q), p_lo = desc_lo(base + SMEM_P);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t par2 = ((uint32_t)j >> 1) & 1u;
        if (!mbar_wait(kv_full(s), par2, abort_flag)) break;
        if (j > 0 && !mbar_wait(s_empty, (uint32_t)(j - 1) & 1u, abort_flag)) break;  // softmax has read S_{j-1}
        tc_fence_after();
        const uint32_t k_lo = desc_lo(base + SMEM_K + s * TILE_BYTES), v_lo = desc_lo(base + SMEM_V + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tmem_s, q_lo + k * 2, k_lo + k * 2, IDESC_S, k != 0);  // 32 bytes of d per step
        tc_commit(s_full);
        if (!mbar_wait(p_full, (uint32_t)j & 1u, abort_flag)) break;  // P_j is in shared memory
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < KT / 16; ++k) {
          // 16 keys per step: P advances 32 bytes inside its 64-key atom (atoms are one tile apart),
          // V advances 16 rows of 128 bytes
          const uint32_t a = p_lo + (uint32_t)((k >> 2) * (TILE_BYTES >> 4) + (k & 3) * 2);
          umma_f16(tmem_o0, a, v_lo + (uint32_t)(k * (16 * 128 >> 4)), IDESC_O, (j | k) != 0);  // O accumulates over tiles
        }
        tc_commit(o_full(s));    // O_j complete (and P_j consumed)
        tc_commit(kv_empty(s));  // K_j / V_j consumed
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + output (one query row per thread)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;           // row within the tile == TMEM lane
    const int qrow = q0 + row;                  // row within the sequence
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const float sc = p.scale * kLog2e;
    uint8_t* prow = smem + SMEM_P + row * 128;  // this row inside a P atom (atoms are TILE_BYTES apart)
    // m_used is the maximum the probabilities are expressed against. It only follows the true running maximum when
    // that has grown by more than 2^8, so the accumulator in TMEM is rescaled rarely (usually once, on the second tile,
    // or never); the final division by l_run makes the result independent of which reference maximum was used.
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < n_tiles; ++j) {
      const int k0 = j * KT;
      // s_full_j also means every earlier MMA of this CTA has completed: P_{j-1} is consumed and O holds tiles < j
      if (!mbar_wait(s_full, (uint32_t)j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32_issue(tmem_s + lane_addr + (uint32_t)(c * 32), sr[c]);
      tmem_ld_wait();
      const bool edge = (k0 + KT > len) || (p.causal && k0 + KT - 1 > q0 + quad * 32);
      if (edge) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = k0 + c * 32 + i;
            if (key >= len || (p.causal && key > qrow)) sr[c][i] = 0xff800000u;  // -inf
          }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sr[c][i]));
      const float m_new = fmaxf(m_used, mx * sc);
      const bool grow = (m_new - m_used > 8.0f) || (m_used == -INFINITY && m_new != -INFINITY);
      if (j == 0) {
        if (grow) m_used = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        const float corr = grow ? ex2(m_used - m_new) : 1.0f;  // 2^-inf = 0 covers a row that had seen no live key yet
        if (grow) m_used = m_new;
        l_run *= corr;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32_issue(tmem_o0 + lane_addr + (uint32_t)(c * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
          tmem_st32(tmem_o0 + lane_addr + (uint32_t)(c * 32), r);
        }
        tmem_st_wait();
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint8_t* atom = prow + (c >> 1) * TILE_BYTES;  // keys 0..63 -> atom 0, 64..127 -> atom 1
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            e[i] = ex2(fmaf(__uint_as_float(sr[c][g8 * 8 + i]), sc, -m_sub));
            rs += e[i];
          }
          uint4 q;
          q.x = pack2<T>(e[0], e[1]);
          q.y = pack2<T>(e[2], e[3]);
          q.z = pack2<T>(e[4], e[5]);
          q.w = pack2<T>(e[6], e[7]);
          const int chunk = (c & 1) * 4 + g8;
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) << 4)) = q;
        }
      }
      l_run += rs;
      tc_fence_before();                                            // S_j read, O rescaled
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P_j visible to the MMA's shared-memory reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_empty);
        mbar_arrive(p_full);
      }
    }
    if (ok && n_tiles > 0) {
      const int last = n_tiles - 1;
      ok = mbar_wait(o_full(last & 1), ((uint32_t)last >> 1) & 1u, abort_flag);
      tc_fence_after();
    }
    if (ok) {
      const float inv = 1.0f / l_run;
      T* op = static_cast<T*>(p.out) + (long long)(tok0 + qrow) * H + h * D;  // 128 contiguous bytes per row
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32_issue(tmem_o0 + lane_addr + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        if (qrow < len) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            uint4 q;
            q.x = pack2<T>(__uint_as_float(r[g8 * 8 + 0]) * inv, __uint_as_float(r[g8 * 8 + 1]) * inv);
            q.y = pack2<T>(__uint_as_float(r[g8 * 8 + 2]) * inv, __uint_as_float(r[g8 * 8 + 3]) * inv);
            q.z = pack2<T>(__uint_as_float(r[g8 * 8 + 4]) * inv, __uint_as_float(r[g8 * 8 + 5]) * inv);
            q.w = pack2<T>(__uint_as_float(r[g8 * 8 + 6]) * inv, __uint_as_float(r[g8 * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(op + c * 32 + g8 * 8) = q;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, (int)TTB_ERR_DEVICE_WAIT);
}

}  // namespace

namespace ttb {

// TTB_ATTN_TC: 0 = never use the tensor-memory kernel, 2 = use it whenever it can run (tests use this to cover ragged
// and causal batches), anything else / unset = let the dispatcher choose by shape. Read on every call.
int attention_tc_mode() {
  const char* e = getenv("TTB_ATTN_TC");
  if (e && e[0] == '0') return 0;
  if (e && e[0] == '2') return 2;
  return 1;
}

// Launches the tcgen05 attention kernel. qkv is [tokens, 3*heads*64] in fp16/bf16; no mask tensor (callers with one use
// the mma.sync kernel). Returns TTB_ERR_UNSUPPORTED when the tensor map cannot be encoded so the caller can fall back.
int attention_tc_launch(ttb_ctx* ctx, int dtype, const void* qkv, int64_t tokens, const int32_t* cu, int64_t B, int64_t max_seqlen,
                        int64_t heads, int causal, float scale, void* out) {
  const int64_t H = heads * D;
  CUtensorMap tm;
  if (!encode_tile_map(&tm, qkv, 2, dtype == TTB_BF16, (uint64_t)tokens, (uint64_t)(3 * H), (uint64_t)(3 * H), 128))
    return TTB_ERR_UNSUPPORTED;
  Params p{out, cu, (int)heads, causal ? 1 : 0, scale, ctx->d_status};
  dim3 grid((unsigned)((max_seqlen + QT - 1) / QT), (unsigned)heads, (unsigned)B);
  static bool configured[64] = {};
  const int dev = ctx->device < 64 ? ctx->device : 63;
  if (!configured[dev]) {
    TTB_CUDA(ctx, cudaFuncSetAttribute(attention_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    TTB_CUDA(ctx, cudaFuncSetAttribute(attention_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured[dev] = true;
  }
  if (dtype == TTB_F16) attention_tc_kernel<__half><<<grid, kThreads, SMEM_BYTES, ctx->stream>>>(tm, p);
  else attention_tc_kernel<__nv_bfloat16><<<grid, kThreads, SMEM_BYTES, ctx->stream>>>(tm, p);
  return launched(ctx, "attention_tc");
}

}  // namespace ttb
