// Tensor-core Linear for sm_100a: out[M,N] = epilogue(sum over passes of A_p[M,K] . W_p[N,K]^T).
//
// One persistent CTA (or CTA pair) per SM, 320 threads in three roles:
//   warp 0      : TMA producer  - cp.async.bulk.tensor loads of 128-byte-swizzled K-major tiles into a
//                 shared-memory ring, completion signalled on "full" mbarriers
//   warp 1      : MMA issuer    - one elected thread issues tcgen05.mma (128 x BN x 32 bytes of K per instruction)
//                 from shared-memory descriptors into a TMEM accumulator; tcgen05.commit releases ring
//                 slots ("empty" mbarriers) and publishes finished accumulators ("tmem_full")
//   warps 2..9  : epilogue      - tcgen05.ld the accumulator (one row per thread), apply scale/bias/activation/
//                 residual in fp32, convert, stage through a swizzled shared-memory tile and TMA-store it
// Two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the MMAs of tile i+1.
//
// Operand kinds: fp16, bf16 (kind::f16), int8 (kind::i8, int32 accumulator) and fp32 read as tf32 (kind::tf32).
// A launch may run up to three passes over K into the same accumulator, each pass reading the first or the second
// of two A maps and of two W maps. That is how operands wider than the tensor core's formats are used at full accuracy:
//   bf16 activations kept as hi + lo planes :  A_hi.W + A_lo.W                       (2 passes)
//   fp32 as three tf32 products             :  A_hi.W_hi + A_lo.W_hi + A_hi.W_lo     (3 passes)
// Small problems (M <= 128 with a long K) are split along K over the CTAs of a cluster: every CTA accumulates its K range
// in its own TMEM, the others hand their partial tile to the first CTA through distributed shared memory, and that CTA
// adds them in rank order and runs the epilogue, so the result does not depend on timing.
// Every mbarrier wait is bounded: on expiry the CTA raises a flag, all roles fall through to the common
// teardown (TMEM is released), and the host sees TTB_ERR_DEVICE_WAIT in the status word.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <unordered_map>

#include "ttb_common.cuh"
#include "ttb_sm100.cuh"

using namespace ttb;
using namespace ttb::sm100;

namespace {

constexpr int BM = 128;          // rows of A per tile == TMEM lanes
constexpr int BK_BYTES = 128;    // bytes of K per ring slot row: one 128-byte swizzle span
constexpr int UMMA_K_BYTES = 32; // K bytes consumed by one tcgen05.mma (16 x 16-bit, 32 x 8-bit, 8 x tf32)
constexpr int kThreads = 320;    // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two per TMEM lane quarter)
constexpr int kMaxSplit = 4;     // CTAs of a cluster that may share one tile's K range (clusters of 6 pack badly into the GPCs:
                                 // 24 of them did not fit the chip at once and the launch took two waves)

// TWO = a pair of CTAs (one cluster of two SMs) computes a 256 x BN tile with cta_group::2 MMAs: each CTA stages its
// own 128 rows of A and its own half (BN/2 rows) of W, so a k-block costs 32 KB of L2->SM traffic per CTA instead of 48.
// SK = split-K over a cluster (BN = 32 only): a shorter ring, plus room for the partial tiles of the other CTAs.
constexpr int kLnMaxTiles = 4;  // kernels with the LayerNorm epilogue: N-tiles of 256 per row, N <= 1024
template <int BN, bool TWO = false, bool SK = false> struct Cfg {
  static constexpr int A_BYTES = BM * BK_BYTES;
  static constexpr int B_BYTES = (TWO ? BN / 2 : BN) * BK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = SK ? 4 : (TWO ? 6 : ((BN == 256) ? 4 : (BN == 128 ? 6 : 8)));
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  // Epilogue staging: per epilogue warp one [32 rows x 128 B] swizzled tile that its TMA stores read (BN >= 64 only).
  static constexpr int STAGING_BYTES = (BN >= 64) ? 8 * 4096 : 0;
  static constexpr int REDUCE_BYTES = SK ? (kMaxSplit - 1) * BM * BN * 4 : 0;  // [slot][column][row] 32-bit words
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + REDUCE_BYTES + BAR_BYTES + 1024;  // + slack for 1024-byte alignment
};

struct GemmParams {
  int M, N, K;             // K in elements, per pass
  int npass;               // 1..3 passes over K into one accumulator
  int pass_a, pass_b;      // bit p set: pass p reads the second A map / the second W map
  void* out;
  long long ldo;
  void* out_lo;            // 16-bit outputs: plane that receives v - round(v) (same pitch as out), or null
  const void* bias;        // OutT[N] or null
  const void* residual;    // OutT[M, ldr] or null
  long long ldr;
  const float* row_scale;  // int8, symmetric: per-row activation scale
  const float* w_scale;    // int8: device scalar, weight scale
  const float* act_qparams;  // int8, affine per tensor: device [scale, zero point]; null selects the symmetric form
  const int* col_sum;        // int8, affine: sum over k of Wq[n, k]
  float* row_absmax;         // int8 kind, or null: [M], receives max |out[m, :]| as stored (atomic maximum; zero before the launch)
  const void* ln_gamma;      // LN kernels: OutT[N], OutT[N], eps
  const void* ln_beta;
  float ln_eps;
  float2* ln_partials;       // LN kernels: [2 * N / 256 slots][ln_rows] {sum, sum of squares} of a row over 128 columns
  int* ln_counters;          // LN kernels: per 128-row block {warps that have published, warps that have read}; all zero between launches
  long long ln_rows;         // rows of the partials array (M rounded up to whole tiles)
  int epilogue;
  int tma_store;           // 1: the output tile goes through shared memory and TMA stores (needs aligned, 16-byte-multiple rows)
  int split_k;             // CTAs per cluster sharing one tile (SK kernels), else 1
  int* status;
};

// 32 lanes x 32 columns of 32-bit accumulators, issued and waited for.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  tmem_ld32_issue(taddr, r);
  tmem_ld_wait();
}

// One 16-byte group of output elements <-> floats: 8 values for the 16-bit types, 4 for fp32.
template <typename OutT> struct Per16 { static constexpr int value = 16 / (int)sizeof(OutT); };
template <typename OutT> __device__ __forceinline__ void unpack16(const uint4& q, float* f);
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& q, float* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& q, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void unpack16<float>(const uint4& q, float* f) {
  f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
}
template <typename OutT> __device__ __forceinline__ uint4 pack16(const float* f);
template <> __device__ __forceinline__ uint4 pack16<__half>(const float* f) {
  uint4 q;
  __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  return q;
}
template <> __device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float* f) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}
template <> __device__ __forceinline__ uint4 pack16<float>(const float* f) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
// What is left of v after rounding it to OutT (the "lo" plane of a two-plane 16-bit value).
template <typename OutT> __device__ __forceinline__ float round_residue(float v) { return v - to_f(from_f<OutT>(v)); }

// Instruction descriptor: accumulator format, operand formats, both operands K-major, N>>3, M>>4.
template <int KIND, int BN, bool TWO = false> __host__ __device__ constexpr uint32_t make_idesc() {
  return (KIND == KIND_I8 ? (2u << 4) | (1u << 7) | (1u << 10)                  // S32 accumulator, signed 8-bit A and B
          : KIND == KIND_TF32 ? (1u << 4) | (2u << 7) | (2u << 10)              // F32 accumulator, TF32 A and B
                              : (1u << 4) | ((uint32_t)KIND << 7) | ((uint32_t)KIND << 10))  // F32 accumulator, F16(0)/BF16(1)
         | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((TWO ? 2 * BM : BM) >> 4) << 24);
}

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 16-bit outputs use the hardware tanh approximation (its error is below their rounding step); fp32 outputs the full one.
template <typename OutT> __device__ __forceinline__ float tanh_out(float x) { return std::is_same<OutT, float>::value ? tanhf(x) : tanh_fast(x); }
template <typename OutT> __device__ __forceinline__ float gelu_out(float x) {
  if (std::is_same<OutT, float>::value) return gelu_tanh(x);  // the fp32 models' exact form
  const float hx = 0.5f * x;  // 0.5x(1 + tanh(0.79788456(x + 0.044715x^3))), regrouped to six operations
  return fmaf(hx, tanh_fast(x * fmaf(x * x, 0.7978845608028654f * 0.044715f, 0.7978845608028654f)), hx);
}

template <typename OutT> __device__ __forceinline__ void load32(const OutT* p, float (&f)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    Vec8<OutT> v;
    v.load(p + i * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[i * 8 + j] = v.v[j];
  }
}

// ---- the kernel -----------------------------------------------------------------------------------
// VAR selects an epilogue variant that costs registers, so that the plain kernels do not carry it:
//   VAR_PLAIN, VAR_TWO_PLANES (16-bit output written as hi + lo planes), VAR_AFFINE (int8 with a per-tensor zero point)
enum { VAR_PLAIN = 0, VAR_TWO_PLANES = 1, VAR_AFFINE = 2 };

template <int BN, int KIND, typename OutT, bool TWO, bool SK, int VAR, bool LN = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
               const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
               const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmO2, const GemmParams p) {
  using C = Cfg<BN, TWO, SK>;
  static_assert(!SK || (BN == 32 && !TWO), "split-K runs on single-CTA 128 x 32 tiles");
  static_assert(!LN || (BN == 256 && !SK && VAR == VAR_PLAIN && sizeof(OutT) == 2), "the LayerNorm epilogue: 16-bit 256-column tiles");
  constexpr int IN_BYTES = (KIND == KIND_I8) ? 1 : (KIND == KIND_TF32 ? 4 : 2);
  constexpr int BK_ELEMS = BK_BYTES / IN_BYTES;
  constexpr uint32_t IDESC = make_idesc<KIND, BN, TWO>();
  constexpr int TILE_M = TWO ? 2 * BM : BM;                      // output rows per tile (per CTA pair when TWO)
  pdl_trigger();  // the next kernel in the stream may start its own set-up; it waits for this grid before touching memory
  const uint32_t rank = (TWO || SK) ? cluster_ctarank() : 0u;    // 0 = the CTA that issues the MMAs (TWO) / runs the epilogue (SK)
  const int group = SK ? p.split_k : (TWO ? 2 : 1);              // CTAs that share one tile
  const int tile0 = (int)blockIdx.x / group;
  const int tile_step = (int)gridDim.x / group;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  const uint32_t tiles = smem_u32(smem);
  uint8_t* staging = smem + C::STAGES * C::STAGE_BYTES;  // 1024-byte aligned: the tile area is a multiple of 1024
  uint32_t* reduce_buf = reinterpret_cast<uint32_t*>(staging + C::STAGING_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::STAGING_BYTES + C::REDUCE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + 2 + a); };
  const uint32_t reduce_bar = bar0 + 8u * (2 * C::STAGES + 4);   // SK: the other CTAs' partial tiles have arrived
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 32) {  // the descriptors are kernel parameters: fetching them does not depend on the previous kernel
    prefetch_tensormap(&tmA0);
    prefetch_tensormap(&tmB0);
    if (p.npass > 1) {
      prefetch_tensormap(&tmA1);
      prefetch_tensormap(&tmB1);
    }
    if (p.tma_store) prefetch_tensormap(&tmO);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), TWO ? 16 : 8);  // one arrival per epilogue warp (of both CTAs when paired)
    }
    mbar_init(reduce_bar, (SK && group > 1) ? (uint32_t)(group - 1) * 128u : 1u);  // every thread of the other CTAs' four working warps
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    if (TWO) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"((uint32_t)C::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      tmem_alloc(smem_u32(tmem_slot), (uint32_t)C::TMEM_COLS);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (TWO || SK) cluster_sync_all();  // the peers' barriers are initialised before anything signals them remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // everything above ran in the shadow of the previous kernel; its results are visible from here on

  const int num_m = (p.M + TILE_M - 1) / TILE_M, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK_ELEMS - 1) / BK_ELEMS;   // k-blocks per pass
  const int total_kb = num_kb * p.npass;
  // this CTA's share of a tile's k-blocks: all of them, or (split-K) one contiguous range per cluster rank
  const int kb_begin = SK ? (int)(((long long)total_kb * rank) / group) : 0;
  const int kb_end = SK ? (int)(((long long)total_kb * (rank + 1)) / group) : total_kb;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
        const int m_blk = tile / num_n, n_blk = tile % num_n;
        int pass = kb_begin / num_kb, kk = kb_begin % num_kb;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const CUtensorMap* ma = ((p.pass_a >> pass) & 1) ? &tmA1 : &tmA0;
          const CUtensorMap* mb = ((p.pass_b >> pass) & 1) ? &tmB1 : &tmB0;
          const uint32_t a_dst = tiles + stage * C::STAGE_BYTES;
          if (TWO) {
            // CTA 0's barrier counts the bytes of both CTAs; only CTA 0 arms it.
            if (rank == 0) mbar_expect_tx(full_bar(stage), 2u * (uint32_t)C::STAGE_BYTES);
            tma_load_2d_pair(a_dst, ma, full_bar(stage), kk * BK_ELEMS, m_blk * TILE_M + (int)rank * BM);
            tma_load_2d_pair(a_dst + C::A_BYTES, mb, full_bar(stage), kk * BK_ELEMS, n_blk * BN + (int)rank * (BN / 2));
          } else {
            mbar_expect_tx(full_bar(stage), (uint32_t)C::STAGE_BYTES);
            tma_load_2d(a_dst, ma, full_bar(stage), kk * BK_ELEMS, m_blk * BM);
            tma_load_2d(a_dst + C::A_BYTES, mb, full_bar(stage), kk * BK_ELEMS, n_blk * BN);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          if (++kk == num_kb) { kk = 0; ++pass; }
        }
      }
      if (!ok) {
        // Gave up: give copies already in flight time to land (they take microseconds) before the CTA's
        // shared memory is released. A fixed, bounded delay; nothing is waited on.
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && (!TWO || rank == 0)) {
      int stage = 0;
      uint32_t phase = 0;
      int acc_iter = 0;
      bool ok = true;
      // Descriptors differ only in the start-address field of their low word, so the loop below advances that
      // word with one add per MMA instead of rebuilding 64-bit descriptors (this single thread's instruction
      // stream is what paces the tensor core).
      const uint32_t a_lo0 = desc_lo(tiles);
      uint32_t a_lo = a_lo0;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step, ++acc_iter) {
        const int acc = acc_iter & 1;
        const uint32_t acc_phase = (uint32_t)(acc_iter >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        uint32_t accumulate = 0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          const uint32_t b_lo = a_lo + (uint32_t)(C::A_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK_BYTES / UMMA_K_BYTES; ++k) {
            umma_ss<KIND, TWO>(d_tmem, a_lo + (uint32_t)(k * (UMMA_K_BYTES >> 4)), b_lo + (uint32_t)(k * (UMMA_K_BYTES >> 4)), IDESC, accumulate);
            accumulate = 1;
          }
          // the slot is free (in both CTAs when paired) once these MMAs have read it
          if (TWO) tc_commit_pair(empty_bar(stage));
          else tc_commit(empty_bar(stage));
          a_lo += (uint32_t)(C::STAGE_BYTES >> 4);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; a_lo = a_lo0; }
        }
        if (ok) {  // accumulator complete: wake the epilogue warps (of both CTAs when paired)
          if (TWO) tc_commit_pair(tfull_bar(acc));
          else tc_commit(tfull_bar(acc));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Two warps share each TMEM lane quarter and split the tile's staged column chunks between them, so one warp's
    // TMEM / shared-memory / store latencies are covered by the other warp on the same scheduler.
    constexpr int EB = (int)sizeof(OutT);
    constexpr int CH = 128 / EB;                 // output columns of one staged chunk: a 128-byte row (64 or 32)
    constexpr int HALVES = CH / 32;              // 32-column TMEM loads per chunk
    constexpr int G16 = 32 * EB / 16;            // 16-byte groups per row of a 32-column half (4 or 8)
    constexpr int P16 = Per16<OutT>::value;      // elements per 16-byte group (8 or 4)
    constexpr int LO_N = (VAR == VAR_TWO_PLANES) ? 8 : 1;  // 16-byte groups of a chunk's second plane kept in registers
    static_assert(VAR != VAR_TWO_PLANES || sizeof(OutT) == 2, "two-plane outputs are 16-bit");
    static_assert(VAR != VAR_AFFINE || KIND == KIND_I8, "the zero-point correction belongs to the int8 kind");
    const int quad = warp & 3;          // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
    const int half = (warp - 2) >> 2;   // which half of the tile's column chunks this warp takes
    const OutT* bias = static_cast<const OutT*>(p.bias);
    const OutT* residual = static_cast<const OutT*>(p.residual);
    OutT* out = static_cast<OutT*>(p.out);
    const float w_scale = (KIND == KIND_I8) ? *p.w_scale : 1.0f;
    constexpr bool affine = (VAR == VAR_AFFINE);
    const float act_scale = affine ? p.act_qparams[0] : 1.0f;
    const int zero_point = affine ? (int)p.act_qparams[1] : 0;
    constexpr bool two_planes = (VAR == VAR_TWO_PLANES);
    const bool vec_ok = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.out_lo) & 15) == 0) &&
                        (!bias || (reinterpret_cast<uintptr_t>(bias) & 15) == 0) &&
                        (!residual || ((p.ldr % 8 == 0) && (reinterpret_cast<uintptr_t>(residual) & 15) == 0));
    const bool use_tma = (BN >= 64) && p.tma_store;
    uint8_t* buf = staging + (warp - 2) * 4096;  // this warp's [32 rows x 128 B] staging tile
    int acc_iter = 0;
    // Pulls a tile's residual rows towards L2 ahead of time, so the epilogue's loads do not each pay a DRAM
    // round trip: lane l touches the 128-byte lines of row l that the tile covers.
    auto prefetch_residual = [&](int t) {
      if (p.epilogue != TTB_EPI_BIAS_RESIDUAL || t >= num_tiles) return;
      const int r = (t / num_n) * TILE_M + (int)((TWO ? rank : 0u) * BM) + quad * 32 + lane, c0 = (t % num_n) * BN;
      if (r >= p.M) return;
      const OutT* rp = residual + (long long)r * p.ldr + c0;
#pragma unroll
      for (int c = 0; c < BN; c += CH)
        if (c0 + c < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + c));
    };
    // Coalesced fetch of a [32 rows x 128 bytes] residual block: 8 lanes per 128-byte row, 4 rows per instruction.
    auto load_residual = [&](uint4 (&dst)[8], int rb, int c0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int grow = rb + i * 4 + (lane >> 3), gcol = c0 + (lane & 7) * P16;
        dst[i] = (grow < p.M && gcol < p.N) ? __ldg(reinterpret_cast<const uint4*>(residual + (long long)grow * p.ldr + gcol))
                                            : make_uint4(0, 0, 0, 0);
      }
    };
    if (!SK) prefetch_residual(tile0);
    auto release_accumulator = [&](int a) {  // one arrival per epilogue warp on the MMA-issuing CTA's barrier
      if (TWO && rank != 0) mbar_arrive_remote(tempty_bar(a), 0);
      else mbar_arrive(tempty_bar(a));
    };
    // accumulator word -> value before bias: int8 dequantised (symmetric per row, or affine per tensor), else as it is
    auto dequant = [&](uint32_t word, float rs, int colsum) -> float {
      if (KIND != KIND_I8) return __uint_as_float(word);
      return (float)((int)word - zero_point * colsum) * rs;
    };
    if constexpr (LN) {
      // ---- bias + residual + LayerNorm. A warp owns 32 rows x 128 columns of the tile (two staged chunks). Pass 1 builds
      // the values (accumulator + bias + residual, rounded to OutT as the separate kernels would store them), keeps them
      // packed in registers, hands the accumulator back and publishes the rows' partial sums; pass 2 normalises with the
      // sums of the whole row and stores through the staging tile and TMA. The N-tiles of a row block are consecutive
      // tiles, so the CTAs that hold them work on them at the same time (the grid is persistent and wholly resident);
      // they meet through global memory: partial sums, then a counter per 128-row block that every warp raises after
      // publishing and waits on (bounded) before reading. A second counter tells the last reader to reset both.
      const OutT* gamma = static_cast<const OutT*>(p.ln_gamma);
      const OutT* beta = static_cast<const OutT*>(p.ln_beta);
      const int warps_per_block = num_n * 8;
      const float inv_n = 1.0f / (float)p.N;
      for (int tile = tile0; tile < num_tiles; tile += tile_step, ++acc_iter) {
        const int m_blk = tile / num_n, n_blk = tile % num_n;
        const int acc = acc_iter & 1;
        const uint32_t acc_phase = (uint32_t)(acc_iter >> 1) & 1u;
        const int row_block = m_blk * (TILE_M / BM) + (int)(TWO ? rank : 0u);  // which 128 rows of the matrix this CTA holds
        const int row_base = row_block * BM + quad * 32;
        const int c_beg = half * 2;
        uint4 res[8];
        load_residual(res, row_base, n_blk * BN + c_beg * CH);  // before the wait
        if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) break;
        tc_fence_after();
        prefetch_residual(tile + tile_step);
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
        uint4 vp[2][2][4];  // [chunk][32-column half][16-byte group]: the values, packed
        float sum = 0.f, sq = 0.f;
#pragma unroll
        for (int ci = 0; ci < 2; ++ci) {
          const int cc = c_beg + ci;
          const int col0 = n_blk * BN + cc * CH;
          if (lane == 0) bulk_wait_read<0>();  // the staging tile may still be read by the previous tile's last store
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3), ch = lane & 7;
            *reinterpret_cast<uint4*>(buf + r * 128 + ((ch ^ (r & 7)) << 4)) = res[i];
          }
          __syncwarp();
          if (ci == 0) load_residual(res, row_base, col0 + CH);  // the second chunk's rows travel during the first
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int colh = col0 + hh * 32;
            uint4 bq[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) bq[g] = __ldg(reinterpret_cast<const uint4*>(bias + colh + g * 8));
            uint32_t r0[32];
            tmem_ld32_issue(taddr + (uint32_t)(cc * CH + hh * 32), r0);
            tmem_ld_wait();
            if (ci == 1 && hh == 1) {  // this warp's share of the accumulator is in registers: hand it back now
              tc_fence_before();
              __syncwarp();
              if (lane == 0) release_accumulator(acc);
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float bb[8], q[8], v[8];
              unpack16<OutT>(bq[g], bb);
              unpack16<OutT>(*reinterpret_cast<const uint4*>(buf + lane * 128 + (((hh * 4 + g) ^ (lane & 7)) << 4)), q);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r0[g * 8 + j]) + bb[j] + q[j];
              vp[ci][hh][g] = pack16<OutT>(v);
              unpack16<OutT>(vp[ci][hh][g], v);  // the statistics are those of the rounded values
#pragma unroll
              for (int j = 0; j < 8; ++j) { sum += v[j]; sq = fmaf(v[j], v[j], sq); }
            }
          }
          __syncwarp();  // every lane has read its residual row out of the staging tile before it is written again
        }
        {
          const long long prow = (long long)row_base + lane;
          p.ln_partials[(long long)(n_blk * 2 + half) * p.ln_rows + prow] = make_float2(sum, sq);
          __syncwarp();
          int* counters = p.ln_counters + 2 * row_block;
          bool arrived = true;
          if (lane == 0) {
            __threadfence();
            atomicAdd(counters, 1);
            const long long t0 = clock64();
            while (ld_acquire_gpu(counters) < warps_per_block) {
              if (*abort_flag || clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                arrived = false;
                break;
              }
              __nanosleep(40);
            }
          }
          if (!__all_sync(0xffffffffu, arrived)) break;
          float tsum = 0.f, tsq = 0.f;
          for (int sl = 0; sl < 2 * num_n; ++sl) {
            const float2 part = __ldcg(p.ln_partials + (long long)sl * p.ln_rows + prow);
            tsum += part.x;
            tsq += part.y;
          }
          sum = tsum;
          sq = tsq;
          __syncwarp();
          if (lane == 0 && atomicAdd(counters + 1, 1) == warps_per_block - 1) {  // the last reader leaves the block's counters at zero
            counters[0] = 0;
            counters[1] = 0;
          }
        }
        const float mean = sum * inv_n;
        const float rstd = rsqrtf(fmaxf(sq * inv_n - mean * mean, 0.f) + p.ln_eps);
        const float shift = -mean * rstd;
#pragma unroll
        for (int ci = 0; ci < 2; ++ci) {
          const int col0 = n_blk * BN + (c_beg + ci) * CH;
          if (lane == 0) bulk_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + hh * 32 + g * 8;
              float v[8], gg[8], bb[8];
              unpack16<OutT>(vp[ci][hh][g], v);
              unpack16<OutT>(__ldg(reinterpret_cast<const uint4*>(gamma + col)), gg);
              unpack16<OutT>(__ldg(reinterpret_cast<const uint4*>(beta + col)), bb);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = fmaf(fmaf(v[j], rstd, shift), gg[j], bb[j]);
              *reinterpret_cast<uint4*>(buf + lane * 128 + (((hh * 4 + g) ^ (lane & 7)) << 4)) = pack16<OutT>(v);
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmO, smem_u32(buf), col0, row_base);
            bulk_commit();
          }
        }
      }
      if (lane == 0) bulk_wait<0>();
      __syncwarp();
    } else {
    for (int tile = tile0; tile < num_tiles; tile += tile_step, ++acc_iter) {
      const int m_blk = tile / num_n, n_blk = tile % num_n;
      const int acc = acc_iter & 1;
      const uint32_t acc_phase = (uint32_t)(acc_iter >> 1) & 1u;
      const int row_base = m_blk * TILE_M + (int)((TWO ? rank : 0u) * BM) + quad * 32;
      const int row = row_base + lane;
      constexpr int kChunks = (BN >= CH) ? BN / CH : 1;
      constexpr int kPerWarp = (kChunks >= 2) ? kChunks / 2 : 1;
      // this warp's chunks of the tile: [c_beg, c_end), clipped to the columns that exist
      const int valid_chunks = min(kChunks, (p.N - n_blk * BN + CH - 1) / CH);
      const int c_beg = (kChunks >= 2) ? half * kPerWarp : 0;
      const int c_end = (kChunks >= 2 || half == 0) ? min(c_beg + kPerWarp, valid_chunks) : 0;
      const bool staged_work = use_tma && c_beg < c_end;
      uint4 res[8];
      if (staged_work && p.epilogue == TTB_EPI_BIAS_RESIDUAL) load_residual(res, row_base, n_blk * BN + c_beg * CH);  // before the wait
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) break;
      tc_fence_after();
      if (!SK) prefetch_residual(tile + tile_step);  // the next tile's rows, a whole mainloop ahead
      const float rs = (KIND != KIND_I8) ? 1.0f : (affine ? act_scale * w_scale : (row < p.M ? p.row_scale[row] * w_scale : 1.0f));
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      if (use_tma || half == 1) {
        if (!staged_work) {  // nothing to do for this warp on this tile: just hand the accumulator back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) release_accumulator(acc);
          continue;
        }
        // ---- one 128-byte-wide chunk of output columns at a time: TMEM -> registers -> (bias, activation, residual) ->
        //      swizzled shared memory tile -> one TMA store per warp. Residual rows are fetched with coalesced 16-byte
        //      loads (8 lanes per 128-byte row) and handed over through the same tile.
        float row_max = 0.f;  // int8 kind with p.row_absmax: largest |value| this thread produced for its row in this tile
#pragma unroll 1
        for (int cc = c_beg; cc < c_end; ++cc) {
          const int col0 = n_blk * BN + cc * CH;
          // the TMA store that last read this warp's staging tile must have finished reading it
          if (lane == 0) bulk_wait_read<0>();
          __syncwarp();
          if (p.epilogue == TTB_EPI_BIAS_RESIDUAL) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3), ch = lane & 7;
              *reinterpret_cast<uint4*>(buf + r * 128 + ((ch ^ (r & 7)) << 4)) = res[i];
            }
            __syncwarp();
            // the next chunk's residual rows travel while this chunk is computed
            if (cc + 1 < c_end) load_residual(res, row_base, col0 + CH);
          }
          uint4 lo_pack[LO_N];  // two-plane outputs: the chunk's "lo" values, kept until the first store has read the tile
          // 32 columns at a time, to keep the live register set small
#pragma unroll
          for (int hh = 0; hh < HALVES; ++hh) {
            const int colh = col0 + hh * 32;
            // 16-bit outputs fetch the half's bias (4 groups) ahead of the TMEM wait; fp32 outputs (8 groups) fetch each
            // group where it is added, to stay within the register budget
            uint4 bq[(EB == 2) ? G16 : 1];
            if (EB == 2 && p.epilogue != TTB_EPI_NONE) {
#pragma unroll
              for (int g = 0; g < G16; ++g)
                bq[g % ((EB == 2) ? G16 : 1)] = (colh + g * P16 < p.N) ? __ldg(reinterpret_cast<const uint4*>(bias + colh + g * P16)) : make_uint4(0, 0, 0, 0);
            }
            uint32_t r0[32];
            tmem_ld32_issue(taddr + (uint32_t)(cc * CH + hh * 32), r0);
            tmem_ld_wait();
            if (hh == HALVES - 1 && cc == c_end - 1) {  // this warp's share of the accumulator is in registers: hand it back now
              tc_fence_before();
              __syncwarp();
              if (lane == 0) release_accumulator(acc);
            }
            float v[32];
            if (affine) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const int4 cs = (colh + g * 4 < p.N) ? __ldg(reinterpret_cast<const int4*>(p.col_sum + colh + g * 4)) : make_int4(0, 0, 0, 0);
                v[g * 4 + 0] = dequant(r0[g * 4 + 0], rs, cs.x);
                v[g * 4 + 1] = dequant(r0[g * 4 + 1], rs, cs.y);
                v[g * 4 + 2] = dequant(r0[g * 4 + 2], rs, cs.z);
                v[g * 4 + 3] = dequant(r0[g * 4 + 3], rs, cs.w);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = dequant(r0[j], rs, 0);
            }
            if (p.epilogue != TTB_EPI_NONE) {
#pragma unroll
              for (int g = 0; g < G16; ++g) {
                float bb[P16];
                if (EB == 2) unpack16<OutT>(bq[g % ((EB == 2) ? G16 : 1)], bb);
                else unpack16<OutT>((colh + g * P16 < p.N) ? __ldg(reinterpret_cast<const uint4*>(bias + colh + g * P16)) : make_uint4(0, 0, 0, 0), bb);
#pragma unroll
                for (int j = 0; j < P16; ++j) v[g * P16 + j] += bb[j];
              }
            }
            if (p.epilogue == TTB_EPI_BIAS_GELU) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_out<OutT>(v[j]);
            } else if (p.epilogue == TTB_EPI_BIAS_TANH) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = tanh_out<OutT>(v[j]);
            } else if (p.epilogue == TTB_EPI_BIAS_RESIDUAL) {
#pragma unroll
              for (int g = 0; g < G16; ++g) {
                float q[P16];
                unpack16<OutT>(*reinterpret_cast<const uint4*>(buf + lane * 128 + (((hh * G16 + g) ^ (lane & 7)) << 4)), q);
#pragma unroll
                for (int j = 0; j < P16; ++j) v[g * P16 + j] += q[j];
              }
            }
            if (KIND == KIND_I8 && p.row_absmax) {
#pragma unroll
              for (int j = 0; j < 32; ++j) row_max = fmaxf(row_max, fabsf(v[j]));
            }
#pragma unroll
            for (int g = 0; g < G16; ++g)
              *reinterpret_cast<uint4*>(buf + lane * 128 + (((hh * G16 + g) ^ (lane & 7)) << 4)) = pack16<OutT>(&v[g * P16]);
            if (two_planes) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = round_residue<OutT>(v[j]);
#pragma unroll
              for (int g = 0; g < G16; ++g) lo_pack[(hh * G16 + g) % LO_N] = pack16<OutT>(&v[g * P16]);
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmO, smem_u32(buf), col0, row_base);
            bulk_commit();
          }
          if (two_planes) {  // second plane through the same staging tile, once the first store has read it
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int g = 0; g < LO_N; ++g)
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((g ^ (lane & 7)) << 4)) = lo_pack[g];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmO2, smem_u32(buf), col0, row_base);
              bulk_commit();
            }
          }
        }
        // rounding to OutT is monotonic, so the maximum of the stored values is the rounded maximum; non-negative floats
        // order like their bit patterns
        if (KIND == KIND_I8 && p.row_absmax && row < p.M)
          atomicMax(reinterpret_cast<int*>(p.row_absmax + row), __float_as_int(to_f(from_f<OutT>(row_max))));
        continue;
      }
      // ---- direct path (narrow tiles or unaligned output): the first warp of each lane quarter walks the tile
      bool gave_up = false;
      float row_max = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), r);
        const int col0 = n_blk * BN + c * 32;
        if (SK && group > 1) {
          // Split-K: ranks > 0 hand their partial tile to rank 0's shared memory ([slot][column][row] words, so a warp's
          // 32 rows of one column are one 128-byte line) and are done; rank 0 adds the slots in rank order.
          const int trow = quad * 32 + lane;
          if (rank != 0) {
            const uint32_t dst = map_to_rank(smem_u32(reduce_buf), 0) + (uint32_t)((((int)rank - 1) * BN * BM + trow) * 4);
#pragma unroll
            for (int j = 0; j < 32; ++j) st_cluster_f32(dst + (uint32_t)(j * BM * 4), __uint_as_float(r[j]));
            mbar_arrive_remote(reduce_bar, 0);  // release at cluster scope: this thread's stores are visible to the waiter
            continue;
          }
          if (!mbar_wait_cluster(reduce_bar, 0, abort_flag)) { gave_up = true; break; }
          for (int s = 0; s < group - 1; ++s) {
            const uint32_t* src = reduce_buf + s * BN * BM + trow;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (KIND == KIND_I8) r[j] = (uint32_t)((int)r[j] + (int)src[j * BM]);
              else r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(src[j * BM]));
            }
          }
        }
        if (row >= p.M || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = dequant(r[j], rs, (affine && col0 + j < p.N) ? p.col_sum[col0 + j] : 0);
        const bool full = vec_ok && (col0 + 32 <= p.N);
        if (p.epilogue != TTB_EPI_NONE) {
          float b[32];
          if (full) load32<OutT>(bias + col0, b);
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) b[j] = (col0 + j < p.N) ? to_f(bias[col0 + j]) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += b[j];
        }
        if (p.epilogue == TTB_EPI_BIAS_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_out<OutT>(v[j]);
        } else if (p.epilogue == TTB_EPI_BIAS_TANH) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = tanh_out<OutT>(v[j]);
        } else if (p.epilogue == TTB_EPI_BIAS_RESIDUAL) {
          const OutT* rp = residual + (long long)row * p.ldr + col0;
          float q[32];
          if (full) load32<OutT>(rp, q);
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) q[j] = (col0 + j < p.N) ? to_f(rp[j]) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += q[j];
        }
        if (KIND == KIND_I8 && p.row_absmax) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) row_max = fmaxf(row_max, fabsf(v[j]));
        }
#pragma unroll 1
        for (int plane = 0; plane < (two_planes ? 2 : 1); ++plane) {
          OutT* dstp = (plane == 0 ? out : static_cast<OutT*>(p.out_lo)) + (long long)row * p.ldo + col0;
          if (plane == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = round_residue<OutT>(v[j]);
          }
          if (full) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              Vec8<OutT> o;
#pragma unroll
              for (int j = 0; j < 8; ++j) o.v[j] = v[i * 8 + j];
              o.store(dstp + i * 8);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dstp[j] = from_f<OutT>(v[j]);
          }
        }
      }
      if (gave_up) break;
      if (KIND == KIND_I8 && p.row_absmax && row < p.M && !(SK && group > 1 && rank != 0))
        atomicMax(reinterpret_cast<int*>(p.row_absmax + row), __float_as_int(to_f(from_f<OutT>(row_max))));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release_accumulator(acc);
    }
    // every TMA store issued by this warp must be complete before its shared memory goes away
    if (use_tma && lane == 0) bulk_wait<0>();
    __syncwarp();
    }
  }

  // ------------------------------------------------------------------ teardown (all roles reach this)
  tc_fence_before();
  __syncthreads();
  if (TWO || SK) cluster_sync_all();  // no CTA leaves while another may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    if (TWO) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    else tmem_dealloc(tmem_base, (uint32_t)C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, (int)TTB_ERR_DEVICE_WAIT);
}

// ---- host side ------------------------------------------------------------------------------------
// Encoded tensor maps are a pure function of (address, shape, pitch, box, element type): weights keep theirs for the life
// of the model and the pool hands activations the same addresses step after step, so they are cached per process.
struct MapKey {
  const void* ptr;
  int64_t rows, k, ld;
  int box_rows, elem_kind;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows && elem_kind == o.elem_kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& m) const {
    size_t h = std::hash<const void*>()(m.ptr);
    auto mix = [&](uint64_t v) { h ^= std::hash<uint64_t>()(v) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix((uint64_t)m.rows);
    mix((uint64_t)m.k);
    mix((uint64_t)m.ld);
    mix(((uint64_t)m.box_rows << 8) | (uint64_t)m.elem_kind);
    return h;
  }
};
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

// 2-D row-major matrix [rows, k] with `ld` elements between rows; box = [box_rows, 128 bytes of k], 128-byte swizzle.
// Used for both operands (K-major tiles) and for the output (32-row x 128-byte store boxes).
// elem_kind: KIND_F16, KIND_BF16, KIND_I8 (one byte) or KIND_TF32 (fp32 words).
int make_map(ttb_ctx* ctx, CUtensorMap* map, int elem_kind, const void* ptr, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  const MapKey key{ptr, rows, k, ld, box_rows, elem_kind};
  {
    std::lock_guard<std::mutex> g(g_map_mu);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *map = it->second;
      return TTB_OK;
    }
  }
  const int es = elem_kind == KIND_I8 ? 1 : (elem_kind == KIND_TF32 ? 4 : 2);
  if (!encode_tile_map(map, ptr, es, elem_kind == KIND_BF16, (uint64_t)rows, (uint64_t)k, (uint64_t)ld, (uint32_t)box_rows))
    return fail(ctx, TTB_ERR_CUDA, "cuTensorMapEncodeTiled failed or is unavailable (rows=%lld k=%lld ld=%lld elem_bytes=%d)", (long long)rows,
                (long long)k, (long long)ld, es);
  std::lock_guard<std::mutex> g(g_map_mu);
  if (g_map_cache.size() >= 16384) g_map_cache.clear();
  g_map_cache.emplace(key, *map);
  return TTB_OK;
}

template <typename OutT> constexpr int out_kind() {
  return std::is_same<OutT, float>::value ? (int)KIND_TF32 : (std::is_same<OutT, __nv_bfloat16>::value ? (int)KIND_BF16 : (int)KIND_F16);
}

struct Operands {
  const void* A;   // [M, K], pitch lda
  const void* A2;  // second A plane or null
  int64_t lda;
  const void* W;   // [N, K] K-major
  const void* W2;  // second W plane or null
};

template <int BN, int KIND, typename OutT, bool TWO, bool SK, int VAR>
int launch_tc(ttb_ctx* ctx, const Operands& op, const GemmParams& p) {
  using C = Cfg<BN, TWO, SK>;
  constexpr int TILE_M = TWO ? 2 * BM : BM;
  constexpr int EA = (int)sizeof(OutT) == 4 ? 4 : 8;  // output elements per 16 bytes
  CUtensorMap tmA0, tmA1, tmB0, tmB1;
  int s = make_map(ctx, &tmA0, KIND, op.A, p.M, p.K, op.lda, BM);
  if (s) return s;
  tmA1 = tmA0;
  if (op.A2 && (s = make_map(ctx, &tmA1, KIND, op.A2, p.M, p.K, op.lda, BM))) return s;
  s = make_map(ctx, &tmB0, KIND, op.W, p.N, p.K, p.K, TWO ? BN / 2 : BN);
  if (s) return s;
  tmB1 = tmB0;
  if (op.W2 && (s = make_map(ctx, &tmB1, KIND, op.W2, p.N, p.K, p.K, TWO ? BN / 2 : BN))) return s;
  GemmParams q = p;
  CUtensorMap tmO = tmA0, tmO2 = tmA0;  // placeholders when the direct-store epilogue is used
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.out_lo) | reinterpret_cast<uintptr_t>(p.bias) |
                           reinterpret_cast<uintptr_t>(p.residual) | reinterpret_cast<uintptr_t>(p.col_sum)) & 15) == 0;
  // The staged epilogue reads bias and residual one 16-byte group at a time, and a TMA store clips a row at 16-byte
  // granularity: with a ragged N it writes zeros into the columns up to the next multiple of 16 bytes. So a ragged N takes
  // this route only without bias/residual and when the caller declared those columns scratch (p.tma_store on entry).
  q.tma_store = (BN >= 64 && aligned16 && p.ldo % EA == 0 && (p.N % EA == 0 || (p.epilogue == TTB_EPI_NONE && p.tma_store && !p.out_lo)) &&
                 (!p.residual || p.ldr % EA == 0)) ? 1 : 0;
  if (q.tma_store) {
    s = make_map(ctx, &tmO, out_kind<OutT>(), p.out, p.M, p.N, p.ldo, 32);
    if (s) return s;
    if (p.out_lo && (s = make_map(ctx, &tmO2, out_kind<OutT>(), p.out_lo, p.M, p.N, p.ldo, 32))) return s;
  }
  auto kern = gemm_tc_kernel<BN, KIND, OutT, TWO, SK, VAR>;
  static bool configured[64] = {};  // per instantiation and device
  static int max_clusters[64] = {};
  const int dev = ctx->device < 64 ? ctx->device : 63;
  if (ctx->device >= 64 || !configured[dev]) {
    TTB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    if (TWO) {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(2 * (unsigned)ctx->sm_count);
      probe.blockDim = dim3(kThreads);
      probe.dynamicSmemBytes = C::SMEM_BYTES;
      cudaLaunchAttribute pa[1];
      pa[0].id = cudaLaunchAttributeClusterDimension;
      pa[0].val.clusterDim.x = 2;
      pa[0].val.clusterDim.y = 1;
      pa[0].val.clusterDim.z = 1;
      probe.attrs = pa;
      probe.numAttrs = 1;
      int n = 0;
      TTB_CUDA(ctx, cudaOccupancyMaxActiveClusters(&n, kern, &probe));
      max_clusters[dev] = n > 0 ? n : 1;
    }
    configured[dev] = true;
  }
  const int64_t num_tiles = ((p.M + TILE_M - 1) / TILE_M) * (int64_t)((p.N + BN - 1) / BN);
  if (!TWO && !SK) {
    const int grid = (int)(num_tiles < ctx->sm_count ? num_tiles : ctx->sm_count);
    cudaError_t e = launch_pdl(kern, dim3((unsigned)grid), dim3(kThreads), C::SMEM_BYTES, ctx->stream, tmA0, tmA1, tmB0, tmB1, tmO, tmO2, q);
    if (e != cudaSuccess) return fail(ctx, TTB_ERR_CUDA, "launch of gemm_tc failed: %s", cudaGetErrorString(e));
    return launched(ctx, "gemm_tc");
  }
  const int group = SK ? p.split_k : 2;
  const int clusters = SK ? (int)num_tiles : (int)(num_tiles < max_clusters[dev] ? num_tiles : max_clusters[dev]);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(group * clusters));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)group;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA0, tmA1, tmB0, tmB1, tmO, tmO2, q);
  if (e != cudaSuccess) return fail(ctx, TTB_ERR_CUDA, "cluster launch of gemm_tc failed: %s", cudaGetErrorString(e));
  return launched(ctx, SK ? "gemm_tc_splitk" : "gemm_tc_pair");
}

// The GEMM whose epilogue is bias + residual + LayerNorm (N a multiple of 256, at most 1024), on the same persistent tile
// schedule as the plain kernels. Returns TTB_ERR_UNSUPPORTED (nothing launched) when its workspace cannot be had right now
// (it would have to grow while the stream is being captured); the caller then runs the product and the LayerNorm as two
// kernels.
constexpr size_t ln_ws_bytes(size_t rows) { return 2 * kLnMaxTiles * rows * sizeof(float2) + (rows / BM) * 2 * sizeof(int); }

int ensure_ln_workspace(ttb_ctx* ctx, size_t rows) {
  if (ctx->ln_ws && ctx->ln_ws_rows >= rows) return TTB_OK;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return TTB_ERR_UNSUPPORTED;
  }
  size_t want = ctx->ln_ws_rows ? ctx->ln_ws_rows : 32768;
  while (want < rows) want *= 2;
  TTB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // nothing may still be using the old one
  if (ctx->ln_ws) cudaFree(ctx->ln_ws);
  ctx->ln_ws = nullptr;
  ctx->ln_ws_rows = 0;
  void* ws = nullptr;
  TTB_CUDA(ctx, cudaMalloc(&ws, ln_ws_bytes(want)));
  TTB_CUDA(ctx, cudaMemset(ws, 0, ln_ws_bytes(want)));
  ctx->ln_ws = ws;
  ctx->ln_ws_rows = want;
  return TTB_OK;
}

template <int KIND, typename OutT, bool TWO>
int launch_tc_ln(ttb_ctx* ctx, const Operands& op, const GemmParams& p) {
  using C = Cfg<256, TWO, false>;
  constexpr int BN = 256;
  constexpr int TILE_M = TWO ? 2 * BM : BM;
  const int64_t num_m = (p.M + TILE_M - 1) / TILE_M;
  const int num_n = p.N / BN;
  const size_t rows = (size_t)num_m * TILE_M;
  int s = ensure_ln_workspace(ctx, rows);
  if (s) return s;
  CUtensorMap tmA0, tmB0, tmO;
  if ((s = make_map(ctx, &tmA0, KIND, op.A, p.M, p.K, op.lda, BM))) return s;
  if ((s = make_map(ctx, &tmB0, KIND, op.W, p.N, p.K, p.K, TWO ? BN / 2 : BN))) return s;
  if ((s = make_map(ctx, &tmO, out_kind<OutT>(), p.out, p.M, p.N, p.ldo, 32))) return s;
  GemmParams q = p;
  q.tma_store = 1;
  q.ln_partials = static_cast<float2*>(ctx->ln_ws);
  q.ln_rows = (long long)ctx->ln_ws_rows;
  q.ln_counters = reinterpret_cast<int*>(static_cast<char*>(ctx->ln_ws) + 2 * kLnMaxTiles * ctx->ln_ws_rows * sizeof(float2));
  auto kern = gemm_tc_kernel<256, KIND, OutT, TWO, false, VAR_PLAIN, true>;
  static int resident[64] = {};  // per instantiation and device: CTAs (single) or CTA pairs (TWO) the device holds at once
  const int dev = ctx->device < 64 ? ctx->device : 63;
  if (ctx->device >= 64 || resident[dev] == 0) {
    TTB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    int n = ctx->sm_count;
    if (TWO) {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(2 * (unsigned)ctx->sm_count);
      probe.blockDim = dim3(kThreads);
      probe.dynamicSmemBytes = C::SMEM_BYTES;
      cudaLaunchAttribute pa[1];
      pa[0].id = cudaLaunchAttributeClusterDimension;
      pa[0].val.clusterDim.x = 2;
      pa[0].val.clusterDim.y = 1;
      pa[0].val.clusterDim.z = 1;
      probe.attrs = pa;
      probe.numAttrs = 1;
      TTB_CUDA(ctx, cudaOccupancyMaxActiveClusters(&n, kern, &probe));
    }
    resident[dev] = n > 0 ? n : 1;
  }
  // Every CTA must be resident: the CTAs that hold one row block wait for one another. Whole row blocks per round also keep
  // the N-tiles of a block in the same round.
  const int64_t num_tiles = num_m * num_n;
  int64_t units = num_tiles < resident[dev] ? num_tiles : (resident[dev] / num_n) * num_n;
  if (units < num_n) return TTB_ERR_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(units * (TWO ? 2 : 1)));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (TWO) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA0, tmA0, tmB0, tmB0, tmO, tmO, q);
  if (e != cudaSuccess) return fail(ctx, TTB_ERR_CUDA, "launch of gemm_tc (LayerNorm epilogue) failed: %s", cudaGetErrorString(e));
  return launched(ctx, "gemm_tc_layernorm");
}

// TTB_GEMM_PAIR: 0 disables the two-CTA variant, 2 uses it for every shape with at least half a wave of pair tiles
// (measurement switches); unset = chosen by shape. TTB_GEMM_SPLITK=0 disables split-K.
int pair_mode() {
  static const int mode = [] {
    const char* e = getenv("TTB_GEMM_PAIR");
    return (e && e[0] == '0') ? 0 : ((e && e[0] == '2') ? 2 : 1);
  }();
  return mode;
}
// TTB_GEMM_SPLITK: 0 disables split-K, 2..6 caps the number of CTAs that share a tile (measurement switch).
int splitk_cap() {
  static const int cap = [] {
    const char* e = getenv("TTB_GEMM_SPLITK");
    if (!e || !e[0]) return kMaxSplit;
    const int v = atoi(e);
    return v <= 1 ? 1 : (v > kMaxSplit ? kMaxSplit : v);
  }();
  return cap;
}

// Clusters of `split` CTAs of the split-K kernel that can be resident on the device at once (cached per device and size).
template <int KIND, typename OutT, int VAR>
int max_resident_clusters(ttb_ctx* ctx, int split) {
  using C = Cfg<32, false, true>;
  static int cached[64][kMaxSplit + 1] = {};
  const int dev = ctx->device < 64 ? ctx->device : 63;
  if (ctx->device < 64 && cached[dev][split] != 0) return cached[dev][split] > 0 ? cached[dev][split] : 0;
  auto kern = gemm_tc_kernel<32, KIND, OutT, false, true, VAR>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t probe = {};
  probe.gridDim = dim3((unsigned)(split * ctx->sm_count));
  probe.blockDim = dim3(kThreads);
  probe.dynamicSmemBytes = C::SMEM_BYTES;
  cudaLaunchAttribute pa[1];
  pa[0].id = cudaLaunchAttributeClusterDimension;
  pa[0].val.clusterDim.x = (unsigned)split;
  pa[0].val.clusterDim.y = 1;
  pa[0].val.clusterDim.z = 1;
  probe.attrs = pa;
  probe.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &probe) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  if (ctx->device < 64) cached[dev][split] = n > 0 ? n : -1;
  return n;
}

template <int KIND, typename OutT, int VAR = VAR_PLAIN>
int pick_tile(ttb_ctx* ctx, const Operands& op, GemmParams& p) {
  // Large problems: CTA pairs on 256 x 256 tiles (less L2->SM traffic per flop). Otherwise the largest single-CTA
  // N-tile that still gives every SM a tile; small problems use narrow tiles to spread over SMs.
  constexpr int IN_BYTES = (KIND == KIND_I8) ? 1 : (KIND == KIND_TF32 ? 4 : 2);
  const int64_t num_m = (p.M + BM - 1) / BM;
  auto tiles = [&](int bn) { return num_m * ((p.N + bn - 1) / bn); };
  const int64_t pair_tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * (int64_t)((p.N + 255) / 256);
  // Measured on B200 in back-to-back launches at M = 18424 (single CTA -> pair, TFLOP/s): N=2304 K=768 1097 -> 1228,
  // N=3072 K=768 1088 -> 1165, N=768 K=3072 1171 -> 1273, but N=768 K=768 789 -> 756: pairs win unless both the
  // mainloop and the row of tiles are short.
  const int64_t k_bytes = (int64_t)p.K * IN_BYTES * p.npass;
  // (same box, bias + residual epilogue: N = K = 768 25.7 us single against 26.3 paired; N = K = 1024, M = 16384 37.1 against 35.8)
  const bool pair_pays = k_bytes >= 4096 || p.N >= 1536 || (k_bytes >= 2048 && p.N >= 1024);
  p.split_k = 1;
  if (pair_mode() && pair_tiles >= ctx->sm_count / 2 && (pair_pays || pair_mode() == 2)) return launch_tc<256, KIND, OutT, true, false, VAR>(ctx, op, p);
  if (tiles(256) >= ctx->sm_count) return launch_tc<256, KIND, OutT, false, false, VAR>(ctx, op, p);
  if (tiles(128) >= ctx->sm_count) return launch_tc<128, KIND, OutT, false, false, VAR>(ctx, op, p);
  if (tiles(64) >= ctx->sm_count / 2) return launch_tc<64, KIND, OutT, false, false, VAR>(ctx, op, p);
  // Fewer 128 x 32 tiles than half the SMs and a mainloop of several k-blocks: share each tile's K range among the CTAs
  // of a cluster so that the weights stream through (nearly) all SMs instead of a few.
  const int64_t t32 = tiles(32);
  const int64_t total_kb = (((int64_t)p.K * IN_BYTES + BK_BYTES - 1) / BK_BYTES) * p.npass;
  // Measured at M = 128 in a replayed graph: K = 3072 (48 k-blocks) 15.6 us in one CTA per tile, 9.0 us split four ways;
  // K = 768 (12 k-blocks) 6.1 us unsplit and no faster split (the launch, the pipeline fill and the epilogue are what is left).
  if (splitk_cap() > 1 && t32 * 2 <= ctx->sm_count && total_kb >= 24) {
    int64_t s = ctx->sm_count / t32;
    if (s > splitk_cap()) s = splitk_cap();
    if (s > total_kb / 2) s = total_kb / 2;  // at least two k-blocks per CTA
    // all clusters must be resident at once (one wave): how many clusters of s CTAs the device holds depends on how
    // they pack into its GPCs
    while (s >= 2 && t32 > max_resident_clusters<KIND, OutT, VAR>(ctx, (int)s)) --s;
    if (s >= 2) {
      p.split_k = (int)s;
      return launch_tc<32, KIND, OutT, false, true, VAR>(ctx, op, p);
    }
  }
  return launch_tc<32, KIND, OutT, false, false, VAR>(ctx, op, p);
}

int check_linear(ttb_ctx* ctx, const char* what, const void* A, const void* W, const void* bias, const void* residual,
                 int64_t M, int64_t N, int64_t K, int epilogue, const void* out, int64_t ldo, int k_align) {
  TTB_REQUIRE(ctx, M >= 0 && N > 0 && K > 0, "%s: bad shape M=%lld N=%lld K=%lld", what, (long long)M, (long long)N, (long long)K);
  TTB_REQUIRE(ctx, M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "%s: dimension too large", what);
  TTB_REQUIRE(ctx, epilogue >= TTB_EPI_NONE && epilogue <= TTB_EPI_BIAS_TANH, "%s: unknown epilogue %d", what, epilogue);
  if (M == 0) return TTB_OK;
  TTB_REQUIRE(ctx, A && W && out, "%s: null pointer", what);
  TTB_REQUIRE(ctx, epilogue == TTB_EPI_NONE || bias, "%s: epilogue %d needs a bias", what, epilogue);
  TTB_REQUIRE(ctx, epilogue != TTB_EPI_BIAS_RESIDUAL || residual, "%s: residual epilogue needs a residual", what);
  TTB_REQUIRE(ctx, K % k_align == 0, "%s: K=%lld must be a multiple of %d (16-byte TMA rows)", what, (long long)K, k_align);
  TTB_REQUIRE(ctx, ldo >= N, "%s: ldo < N", what);
  TTB_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) % 16 == 0, "%s: operands must be 16-byte aligned", what);
  return TTB_OK;
}

// Zero fill that takes part in programmatic dependent launch: it returns only after the kernel ahead of it has completed,
// so a kernel that waits for this one is ordered after that one too.
__global__ void __launch_bounds__(256) zero_floats_kernel(float* dst, int64_t n) {
  pdl_trigger();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = 0.f;
}

int linear_int8_common(ttb_ctx* ctx, const char* what, int out_dtype, const int8_t* Aq, const float* row_scale, const float* act_qparams,
                       const int8_t* Wq, const float* w_scale, const int32_t* col_sum, const void* bias, const void* residual, int64_t ldr,
                       int64_t M, int64_t N, int64_t K, int epilogue, void* out, int64_t ldo, float* row_absmax = nullptr) {
  TTB_REQUIRE(ctx, out_dtype == TTB_F16 || out_dtype == TTB_BF16, "%s: output dtype must be F16 or BF16", what);
  int s = check_linear(ctx, what, Aq, Wq, bias, residual, M, N, K, epilogue, out, ldo, 16);
  if (s || M == 0) return s;
  TTB_REQUIRE(ctx, (row_scale || act_qparams) && w_scale, "%s: null scale pointer", what);
  TTB_REQUIRE(ctx, !act_qparams || col_sum, "%s: the affine form needs the weight's column sums", what);
  DeviceGuard g(ctx->device);
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.npass = 1;
  p.out = out; p.ldo = ldo; p.bias = bias; p.residual = residual; p.ldr = ldr;
  p.row_scale = row_scale; p.w_scale = w_scale; p.act_qparams = act_qparams; p.col_sum = col_sum;
  p.epilogue = epilogue; p.split_k = 1; p.status = ctx->d_status;
  if (row_absmax) {  // zero-filled by a kernel of its own, so that the launches stay one programmatic-dependency chain
    const int64_t n4 = (M + 3) / 4;
    launch_pdl(zero_floats_kernel, dim3((unsigned)std::min<int64_t>((n4 + 255) / 256, 1024)), dim3(256), 0, ctx->stream, row_absmax, M);
    p.row_absmax = row_absmax;
  }
  const Operands op{Aq, nullptr, K, Wq, nullptr};
  if (act_qparams) {
    if (out_dtype == TTB_F16) return pick_tile<KIND_I8, __half, VAR_AFFINE>(ctx, op, p);
    return pick_tile<KIND_I8, __nv_bfloat16, VAR_AFFINE>(ctx, op, p);
  }
  if (out_dtype == TTB_F16) return pick_tile<KIND_I8, __half>(ctx, op, p);
  return pick_tile<KIND_I8, __nv_bfloat16>(ctx, op, p);
}

// ---- weight re-layout -----------------------------------------------------------------------------
// dst[n, k] = convert(src[k, n])  (or src[n, k] when it is already [N,K])
template <typename S, typename D>
__global__ void __launch_bounds__(256)
prepack_kernel(const S* __restrict__ src, int src_is_nk, int K, int N, D* __restrict__ dst) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;  // 32 x 8
  if (src_is_nk) {
    for (int r = ty; r < 32; r += 8) {
      const int n = n0 + r, k = k0 + tx;
      if (n < N && k < K) dst[(int64_t)n * K + k] = from_f<D>(to_f(src[(int64_t)n * K + k]));
    }
    return;
  }
  for (int r = ty; r < 32; r += 8) {
    const int k = k0 + r, n = n0 + tx;
    tile[r][tx] = (k < K && n < N) ? to_f(src[(int64_t)k * N + n]) : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int n = n0 + r, k = k0 + tx;
    if (n < N && k < K) dst[(int64_t)n * K + k] = from_f<D>(tile[tx][r]);
  }
}

template <typename S>
__global__ void __launch_bounds__(256) absmax_kernel(const S* __restrict__ src, int64_t n, float* __restrict__ amax) {
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(to_f(src[i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));  // non-negative floats order as ints
}

__global__ void amax_to_scale_kernel(float* s) { *s = (*s > 0.f) ? *s / 127.0f : 1.0f; }

template <typename S>
__global__ void __launch_bounds__(256)
prepack_int8_kernel(const S* __restrict__ src, int src_is_nk, int K, int N, const float* __restrict__ scale, int8_t* __restrict__ dst) {
  const float sc = *scale;
  const int64_t n_el = (int64_t)K * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_el; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / K, k = i % K;  // destination order
    const float w = to_f(src_is_nk ? src[i] : src[k * N + n]);
    float q = rintf(w / sc);
    q = fminf(fmaxf(q, -127.f), 127.f);
    dst[i] = (int8_t)q;
  }
}

// torch's per-tensor symmetric qint8 rule (MinMaxObserver): scale = max|W| / 127.5, q = clamp(rint(W * (1 / scale)), -128, 127).
__global__ void amax_to_scale_torch_kernel(float* s) {
  const float sc = *s / 127.5f;
  *s = fmaxf(sc, 1.1920928955078125e-07f);
}
template <typename S>
__global__ void __launch_bounds__(256)
prepack_int8_torch_kernel(const S* __restrict__ src, int src_is_nk, int K, int N, const float* __restrict__ scale, int8_t* __restrict__ dst) {
  const float inv = 1.0f / *scale;
  const int64_t n_el = (int64_t)K * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_el; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / K, k = i % K;  // destination order
    const float w = to_f(src_is_nk ? src[i] : src[k * N + n]);
    dst[i] = (int8_t)fminf(fmaxf(rintf(w * inv), -128.f), 127.f);
  }
}
// col_sum[n] = sum over k of Wq[n, k]: one warp per output row.
__global__ void __launch_bounds__(256) int8_row_sum_kernel(const int8_t* __restrict__ wq, int K, int N, int32_t* __restrict__ col_sum) {
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= N) return;
  int acc = 0;
  for (int k = lane; k < K; k += 32) acc += wq[(int64_t)n * K + k];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) col_sum[n] = acc;
}

// fp32 -> two tf32-representable planes: hi = x rounded to 10 mantissa bits, lo = (x - hi) rounded likewise. hi + lo carries
// 21 of x's 24 significant bits, which is what three tf32 products recover.
__device__ __forceinline__ float round_tf32(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}
__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ hi, float* __restrict__ lo) {
  // x may alias hi (in-place split of a weight): each element is read before it is written, by the same thread
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      float4 h, l;
      h.x = round_tf32(v.x); h.y = round_tf32(v.y); h.z = round_tf32(v.z); h.w = round_tf32(v.w);
      l.x = round_tf32(v.x - h.x); l.y = round_tf32(v.y - h.y); l.z = round_tf32(v.z - h.z); l.w = round_tf32(v.w - h.w);
      *reinterpret_cast<float4*>(hi + i) = h;
      *reinterpret_cast<float4*>(lo + i) = l;
    } else {
      for (int64_t j = i; j < n; ++j) {
        const float v = x[j], h = round_tf32(v);
        hi[j] = h;
        lo[j] = round_tf32(v - h);
      }
    }
  }
}

}  // namespace

// =================================================================================================
extern "C" int ttb_linear_ex(ttb_ctx* ctx, const ttb_linear_args* a) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, a != nullptr, "linear_ex: null argument block");
  const int dt = a->dtype, odt = a->out_dtype;
  TTB_REQUIRE(ctx, dt == TTB_F16 || dt == TTB_BF16 || dt == TTB_F32, "linear_ex: operand dtype must be F16, BF16 or F32");
  TTB_REQUIRE(ctx, odt == dt || (odt == TTB_F32 && dt != TTB_F32), "linear_ex: the output is of the operand dtype, or F32 for 16-bit operands");
  TTB_REQUIRE(ctx, !a->W2 || (a->A2 && dt == TTB_F32), "linear_ex: a second weight plane belongs to the three-pass fp32 form (A, A2, W, W2)");
  TTB_REQUIRE(ctx, !a->out_lo || odt == TTB_BF16, "linear_ex: the second output plane exists for BF16 outputs only");
  const int pad_scratch = (a->epilogue & TTB_EPI_FLAG_ROW_PADDING_IS_SCRATCH) ? 1 : 0;
  const int epilogue = a->epilogue & ~TTB_EPI_FLAG_ROW_PADDING_IS_SCRATCH;
  const int k_align = dt == TTB_F32 ? 4 : 8;
  int s = check_linear(ctx, "linear", a->A, a->W, a->bias, a->residual, a->M, a->N, a->K, epilogue, a->out, a->ldo, k_align);
  if (s || a->M == 0) return s;
  TTB_REQUIRE(ctx, a->lda >= a->K && a->lda % k_align == 0, "linear: lda must be >= K and a multiple of %d", k_align);
  TTB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(a->A2) | reinterpret_cast<uintptr_t>(a->W2)) & 15) == 0, "linear: operands must be 16-byte aligned");
  DeviceGuard g(ctx->device);
  GemmParams p{};
  p.M = (int)a->M; p.N = (int)a->N; p.K = (int)a->K;
  p.npass = a->W2 ? 3 : (a->A2 ? 2 : 1);
  p.pass_a = a->A2 ? 2 : 0;   // passes: (A, W), (A2, W), (A, W2): bit 1 of pass_a, bit 2 of pass_b
  p.pass_b = a->W2 ? 4 : 0;
  p.out = a->out; p.ldo = a->ldo; p.out_lo = a->out_lo;
  p.bias = a->bias; p.residual = a->residual; p.ldr = a->ldr;
  p.epilogue = epilogue; p.tma_store = pad_scratch; p.split_k = 1; p.status = ctx->d_status;
  const Operands op{a->A, a->A2, a->lda, a->W, a->W2};
  if (dt == TTB_F32) return pick_tile<KIND_TF32, float>(ctx, op, p);
  if (dt == TTB_F16) return odt == TTB_F32 ? pick_tile<KIND_F16, float>(ctx, op, p) : pick_tile<KIND_F16, __half>(ctx, op, p);
  if (odt == TTB_F32) return pick_tile<KIND_BF16, float>(ctx, op, p);
  if (a->out_lo) return pick_tile<KIND_BF16, __nv_bfloat16, VAR_TWO_PLANES>(ctx, op, p);
  return pick_tile<KIND_BF16, __nv_bfloat16>(ctx, op, p);
}

extern "C" int ttb_linear(ttb_ctx* ctx, int dtype, const void* A, int64_t lda, const void* Wp, const void* bias,
                          const void* residual, int64_t ldr, int64_t M, int64_t N, int64_t K, int epilogue, void* out,
                          int64_t ldo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "linear: dtype must be F16 or BF16 (ttb_linear_ex takes F32)");
  ttb_linear_args a{};
  a.dtype = dtype; a.out_dtype = dtype;
  a.A = A; a.lda = lda; a.W = Wp;
  a.bias = bias; a.residual = residual; a.ldr = ldr;
  a.M = M; a.N = N; a.K = K; a.epilogue = epilogue;
  a.out = out; a.ldo = ldo;
  return ttb_linear_ex(ctx, &a);
}

extern "C" int ttb_layernorm(ttb_ctx* ctx, int dtype, const void* in, void* out, const void* gamma, const void* beta, int64_t M, int64_t N,
                             float eps);

// TTB_GEMM_LN (read at every call): unset or 0 = the product and the LayerNorm run as two kernels; 1 = one kernel for Linears
// with a long mainloop (K >= 2048); 2 = one kernel whenever the shape allows. Off by default: the one-kernel form makes the
// CTAs that hold one row block wait for one another through global memory, which needs the whole grid resident at once.
// That holds for one context on a device, but two contexts running such kernels on one device at the same time could
// each hold SMs the other is waiting for (the waits are bounded: the calls would end with TTB_ERR_DEVICE_WAIT), and the
// measured gain is under one per cent of the benchmark step.
static int fused_ln_mode() {
  const char* e = getenv("TTB_GEMM_LN");
  return (e && e[0] >= '1' && e[0] <= '2') ? e[0] - '0' : 0;
}

extern "C" int ttb_linear_layernorm(ttb_ctx* ctx, int dtype, const void* A, int64_t lda, const void* Wp, const void* bias,
                                    const void* residual, int64_t ldr, const void* gamma, const void* beta, float eps, int64_t M, int64_t N,
                                    int64_t K, void* out, int64_t ldo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "linear_layernorm: dtype must be F16 or BF16");
  int s = check_linear(ctx, "linear_layernorm", A, Wp, bias, residual, M, N, K, TTB_EPI_BIAS_RESIDUAL, out, ldo, 8);
  if (s || M == 0) return s;
  TTB_REQUIRE(ctx, gamma && beta, "linear_layernorm: null LayerNorm parameters");
  TTB_REQUIRE(ctx, ldo == N, "linear_layernorm: the output rows must be dense (ldo == N)");
  TTB_REQUIRE(ctx, lda >= K && lda % 8 == 0, "linear_layernorm: lda must be >= K and a multiple of 8");
  const bool aligned = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Wp) | reinterpret_cast<uintptr_t>(bias) |
                         reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta) |
                         reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  // Below about a thousand rows the narrow-tile (and split-K) kernels plus the one-round-trip LayerNorm are faster than
  // N / 256 CTAs walking the whole K range.
  // and with a short mainloop (K < 2048) the kernel runs at the speed of its epilogue, which the exchange of row sums
  // lengthens by more than the separate LayerNorm costs (measured at M = 18424, N = 768: K = 768 40.2 us in one kernel
  // against 25.6 + 12.5; K = 3072 72.1 against 67.6 + 12.5).
  const int mode = fused_ln_mode();
  if (mode && aligned && N % 256 == 0 && N / 256 <= kLnMaxTiles && M >= 1024 && (K >= 2048 || mode == 2) && ldr % 8 == 0 && M < (1ll << 31) &&
      K < (1ll << 31)) {
    DeviceGuard g(ctx->device);
    GemmParams p{};
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.npass = 1;
    p.out = out; p.ldo = ldo; p.bias = bias; p.residual = residual; p.ldr = ldr;
    p.epilogue = TTB_EPI_BIAS_RESIDUAL; p.split_k = 1; p.status = ctx->d_status;
    p.ln_gamma = gamma; p.ln_beta = beta; p.ln_eps = eps;
    const Operands op{A, nullptr, lda, Wp, nullptr};
    // CTA pairs where the plain kernel would use them too: a long mainloop (see pick_tile)
    const bool pair = pair_mode() && K * 2 >= 4096 && ((M + 2 * BM - 1) / (2 * BM)) * (N / 256) >= ctx->sm_count / 2;
    if (dtype == TTB_F16) s = pair ? launch_tc_ln<KIND_F16, __half, true>(ctx, op, p) : launch_tc_ln<KIND_F16, __half, false>(ctx, op, p);
    else s = pair ? launch_tc_ln<KIND_BF16, __nv_bfloat16, true>(ctx, op, p) : launch_tc_ln<KIND_BF16, __nv_bfloat16, false>(ctx, op, p);
    if (s != TTB_ERR_UNSUPPORTED) return s;
  }
  s = ttb_linear(ctx, dtype, A, lda, Wp, bias, residual, ldr, M, N, K, TTB_EPI_BIAS_RESIDUAL, out, ldo);
  if (s) return s;
  return ttb_layernorm(ctx, dtype, out, out, gamma, beta, M, N, eps);
}

extern "C" int ttb_linear_int8(ttb_ctx* ctx, int out_dtype, const int8_t* Aq, const float* row_scale, const int8_t* Wq,
                               const float* w_scale, const void* bias, const void* residual, int64_t ldr, int64_t M,
                               int64_t N, int64_t K, int epilogue, void* out, int64_t ldo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M == 0 || row_scale != nullptr, "linear_int8: null scale pointer");
  return linear_int8_common(ctx, "linear_int8", out_dtype, Aq, row_scale, nullptr, Wq, w_scale, nullptr, bias, residual, ldr, M, N, K, epilogue, out,
                            ldo);
}

extern "C" int ttb_linear_int8_rowmax(ttb_ctx* ctx, int out_dtype, const int8_t* Aq, const float* row_scale, const int8_t* Wq,
                                      const float* w_scale, const void* bias, const void* residual, int64_t ldr, int64_t M, int64_t N,
                                      int64_t K, int epilogue, void* out, int64_t ldo, float* row_absmax) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M == 0 || (row_scale != nullptr && row_absmax != nullptr), "linear_int8_rowmax: null scale or maximum pointer");
  return linear_int8_common(ctx, "linear_int8_rowmax", out_dtype, Aq, row_scale, nullptr, Wq, w_scale, nullptr, bias, residual, ldr, M, N, K, epilogue,
                            out, ldo, row_absmax);
}

extern "C" int ttb_linear_int8_affine(ttb_ctx* ctx, int out_dtype, const int8_t* Aq, const float* act_qparams, const int8_t* Wq,
                                      const float* w_scale, const int32_t* col_sum, const void* bias, const void* residual, int64_t ldr,
                                      int64_t M, int64_t N, int64_t K, int epilogue, void* out, int64_t ldo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, M == 0 || (act_qparams != nullptr && col_sum != nullptr), "linear_int8_affine: null quantisation parameters");
  return linear_int8_common(ctx, "linear_int8_affine", out_dtype, Aq, nullptr, act_qparams, Wq, w_scale, col_sum, bias, residual, ldr, M, N, K,
                            epilogue, out, ldo);
}

extern "C" int ttb_prepack_weight(ttb_ctx* ctx, int src_dtype, const void* src, int src_is_nk, int64_t K, int64_t N,
                                  int dst_dtype, void* dst) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, K > 0 && N > 0 && K < (1ll << 31) && N < (1ll << 31), "prepack_weight: bad shape");
  TTB_REQUIRE(ctx, src && dst, "prepack_weight: null pointer");
  TTB_REQUIRE(ctx, dst_dtype == TTB_F16 || dst_dtype == TTB_BF16 || dst_dtype == TTB_F32, "prepack_weight: bad destination dtype");
  DeviceGuard g(ctx->device);
  dim3 grid((unsigned)((K + 31) / 32), (unsigned)((N + 31) / 32));
  TTB_REQUIRE(ctx, grid.y <= 65535, "prepack_weight: N too large");
#define PREPACK(S, D) prepack_kernel<S, D><<<grid, 256, 0, ctx->stream>>>((const S*)src, src_is_nk, (int)K, (int)N, (D*)dst)
  TTB_DISPATCH_FLOAT(ctx, src_dtype, S, {
    if (dst_dtype == TTB_F16) PREPACK(S, __half);
    else if (dst_dtype == TTB_BF16) PREPACK(S, __nv_bfloat16);
    else PREPACK(S, float);
  });
#undef PREPACK
  return launched(ctx, "prepack_weight");
}

extern "C" int ttb_prepack_weight_int8(ttb_ctx* ctx, int src_dtype, const void* src, int src_is_nk, int64_t K, int64_t N,
                                       int8_t* dst, float* scale_out) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, K > 0 && N > 0, "prepack_weight_int8: bad shape");
  TTB_REQUIRE(ctx, src && dst && scale_out, "prepack_weight_int8: null pointer");
  DeviceGuard g(ctx->device);
  TTB_CUDA(ctx, cudaMemsetAsync(scale_out, 0, sizeof(float), ctx->stream));
  const int64_t n = K * N;
  const int grid = (int)((n + 255) / 256 < (int64_t)ctx->sm_count * 8 ? (n + 255) / 256 : (int64_t)ctx->sm_count * 8);
  TTB_DISPATCH_FLOAT(ctx, src_dtype, S, {
    absmax_kernel<S><<<grid, 256, 0, ctx->stream>>>((const S*)src, n, scale_out);
    amax_to_scale_kernel<<<1, 1, 0, ctx->stream>>>(scale_out);
    prepack_int8_kernel<S><<<grid, 256, 0, ctx->stream>>>((const S*)src, src_is_nk, (int)K, (int)N, scale_out, dst);
  });
  ctx->launches.fetch_add(2);
  return launched(ctx, "prepack_weight_int8");
}

extern "C" int ttb_prepack_weight_int8_affine(ttb_ctx* ctx, int src_dtype, const void* src, int src_is_nk, int64_t K, int64_t N, int8_t* dst,
                                              float* scale_out, int32_t* col_sum_out) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, K > 0 && N > 0 && K < (1ll << 31) && N < (1ll << 31), "prepack_weight_int8_affine: bad shape");
  TTB_REQUIRE(ctx, src && dst && scale_out && col_sum_out, "prepack_weight_int8_affine: null pointer");
  DeviceGuard g(ctx->device);
  TTB_CUDA(ctx, cudaMemsetAsync(scale_out, 0, sizeof(float), ctx->stream));
  const int64_t n = K * N;
  const int grid = (int)((n + 255) / 256 < (int64_t)ctx->sm_count * 8 ? (n + 255) / 256 : (int64_t)ctx->sm_count * 8);
  TTB_DISPATCH_FLOAT(ctx, src_dtype, S, {
    absmax_kernel<S><<<grid, 256, 0, ctx->stream>>>((const S*)src, n, scale_out);
    amax_to_scale_torch_kernel<<<1, 1, 0, ctx->stream>>>(scale_out);
    prepack_int8_torch_kernel<S><<<grid, 256, 0, ctx->stream>>>((const S*)src, src_is_nk, (int)K, (int)N, scale_out, dst);
  });
  int8_row_sum_kernel<<<(unsigned)((N + 7) / 8), 256, 0, ctx->stream>>>(dst, (int)K, (int)N, col_sum_out);
  ctx->launches.fetch_add(3);
  return launched(ctx, "prepack_weight_int8_affine");
}

extern "C" int ttb_split_tf32(ttb_ctx* ctx, const float* x, int64_t n, float* hi, float* lo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, n >= 0, "split_tf32: negative size");
  if (n == 0) return TTB_OK;
  TTB_REQUIRE(ctx, x && hi && lo, "split_tf32: null pointer");
  TTB_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 15) == 0,
              "split_tf32: pointers must be 16-byte aligned");
  DeviceGuard g(ctx->device);
  const int64_t want = (n / 4 + 255) / 256 + 1;
  const int grid = (int)(want < (int64_t)ctx->sm_count * 16 ? want : (int64_t)ctx->sm_count * 16);
  split_tf32_kernel<<<grid, 256, 0, ctx->stream>>>(x, n, hi, lo);
  return launched(ctx, "split_tf32");
}
