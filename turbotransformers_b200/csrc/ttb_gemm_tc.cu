// Tensor-core Linear for sm_100a: out[M,N] = epilogue(A[M,K] . W[N,K]^T).
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      : TMA producer  - cp.async.bulk.tensor loads of 128-byte-swizzled K-major tiles into a
//                 shared-memory ring, completion signalled on "full" mbarriers
//   warp 1      : MMA issuer    - one elected thread issues tcgen05.mma (128 x BN x 16/32 per instruction)
//                 from shared-memory descriptors into a TMEM accumulator; tcgen05.commit releases ring
//                 slots ("empty" mbarriers) and publishes finished accumulators ("tmem_full")
//   warps 2..5  : epilogue      - tcgen05.ld the accumulator (one row per thread), apply scale/bias/activation/
//                 residual in fp32, convert, stage through a swizzled shared-memory tile and TMA-store it
// Two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the MMAs of tile i+1.
// Every mbarrier wait is bounded: on expiry the CTA raises a flag, all roles fall through to the common
// teardown (TMEM is released), and the host sees TTB_ERR_DEVICE_WAIT in the status word.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "ttb_common.cuh"

using namespace ttb;

namespace {

constexpr int BM = 128;          // rows of A per tile == TMEM lanes
constexpr int BK_BYTES = 128;    // bytes of K per ring slot row: one 128-byte swizzle span
constexpr int UMMA_K_BYTES = 32; // K bytes consumed by one tcgen05.mma (16 x 16-bit, 32 x 8-bit)
constexpr int kThreads = 320;    // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two per TMEM lane quarter)
constexpr long long kWaitCycles = 4000000000LL;  // about two seconds of SM clock

enum { KIND_F16 = 0, KIND_BF16 = 1, KIND_I8 = 2 };

// TWO = a pair of CTAs (one cluster of two SMs) computes a 256 x BN tile with cta_group::2 MMAs: each CTA stages its
// own 128 rows of A and its own half (BN/2 rows) of W, so a k-block costs 32 KB of L2->SM traffic per CTA instead of 48.
template <int BN, bool TWO = false> struct Cfg {
  static constexpr int A_BYTES = BM * BK_BYTES;
  static constexpr int B_BYTES = (TWO ? BN / 2 : BN) * BK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = TWO ? 6 : ((BN == 256) ? 4 : (BN == 128 ? 6 : 8));
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  // Epilogue staging: per epilogue warp one [32 rows x 128 B] swizzled tile that its TMA stores read (BN >= 64 only).
  static constexpr int STAGING_BYTES = (BN >= 64) ? 8 * 4096 : 0;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES + 1024;  // + slack for 1024-byte alignment
};

struct GemmParams {
  int M, N, K;             // K in elements
  void* out;
  long long ldo;
  const void* bias;        // OutT[N] or null
  const void* residual;    // OutT[M, ldr] or null
  long long ldr;
  const float* row_scale;  // int8: per-row activation scale
  const float* w_scale;    // int8: device scalar, weight scale
  int epilogue;
  int tma_store;           // 1: the output tile goes through shared memory and TMA stores (needs aligned, 16-byte-multiple rows)
  int* status;
};

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false (and raises the CTA-wide abort flag) when the limit expires or another
// role has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int KIND>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (KIND == KIND_I8) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// ---- two-CTA (cluster of 2) variants --------------------------------------------------------------
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared-window address: "same offset in CTA 0"

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t local_bar, uint32_t target_rank) {
  asm volatile(
      "{\n"
      ".reg .b32 ra;\n"
      "mapa.shared::cluster.u32 ra, %0, %1;\n"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n"
      "}\n" ::"r"(local_bar),
      "r"(target_rank)
      : "memory");
}
// Tile load issued by either CTA of the pair into its own shared memory; the bytes are counted on CTA 0's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar & kPeerBitMask), "r"(x), "r"(y)
      : "memory");
}
// Arrives (once the MMAs issued so far have completed) on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
               : "memory");
}
template <int KIND>
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (KIND == KIND_I8) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// MMA with both shared-memory descriptors given as (low word, shared high word).
template <int KIND, bool TWO>
__device__ __forceinline__ void umma_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                        uint32_t accumulate) {
#define TTB_UMMA_ASM(GROUP, KINDSTR)                                                        \
  asm volatile(                                                                             \
      "{\n"                                                                                 \
      ".reg .pred p;\n"                                                                     \
      ".reg .b64 da, db;\n"                                                                 \
      "setp.ne.b32 p, %5, 0;\n"                                                             \
      "mov.b64 da, {%1, %3};\n"                                                             \
      "mov.b64 db, {%2, %3};\n"                                                             \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], da, db, %4, p;\n"           \
      "}\n" ::"r"(d_tmem),                                                                  \
      "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)                       \
      : "memory")
  if (KIND == KIND_I8) {
    if (TWO) TTB_UMMA_ASM("2", "i8");
    else TTB_UMMA_ASM("1", "i8");
  } else {
    if (TWO) TTB_UMMA_ASM("2", "f16");
    else TTB_UMMA_ASM("1", "f16");
  }
#undef TTB_UMMA_ASM
}

// 32 lanes x 32 columns of 32-bit accumulators: thread t of the warp receives row (lane base + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// TMA store of a [32 rows x 128 B] swizzled shared-memory tile to the output matrix; rows/columns outside the
// matrix are clipped by the hardware. Completion is tracked per issuing thread in bulk groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

template <typename OutT> __device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]);
template <> __device__ __forceinline__ void unpack8<__half>(const uint4& q, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <typename OutT> __device__ __forceinline__ uint4 pack8(const float* f);
template <> __device__ __forceinline__ uint4 pack8<__half>(const float* f) {
  uint4 q;
  __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  return q;
}
template <> __device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float* f) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes, laid out by TMA
// with the 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO); LBO is not used by this layout.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading-dimension byte offset (ignored)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride-dimension byte offset
  d |= (uint64_t)1 << 46;                        // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                        // layout: 128-byte swizzle
  return d;
}

// Instruction descriptor: accumulator format, operand formats, both operands K-major, N>>3, M>>4.
template <int KIND, int BN, bool TWO = false> __host__ __device__ constexpr uint32_t make_idesc() {
  return (KIND == KIND_I8 ? (2u << 4) | (1u << 7) | (1u << 10)            // S32 accum, signed 8-bit A and B
                          : (1u << 4) | ((uint32_t)KIND << 7) | ((uint32_t)KIND << 10))  // F32 accum, F16(0)/BF16(1)
         | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((TWO ? 2 * BM : BM) >> 4) << 24);
}

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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
template <int BN, int KIND, typename OutT, bool TWO>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmO, const GemmParams p) {
  using C = Cfg<BN, TWO>;
  constexpr int BK_ELEMS = (KIND == KIND_I8) ? BK_BYTES : BK_BYTES / 2;
  constexpr uint32_t IDESC = make_idesc<KIND, BN, TWO>();
  constexpr int TILE_M = TWO ? 2 * BM : BM;                      // output rows per tile (per CTA pair when TWO)
  pdl_trigger();  // the next kernel in the stream may start its own set-up; it waits for this grid before touching memory
  const uint32_t rank = TWO ? cluster_ctarank() : 0u;            // 0 = the CTA that issues the MMAs
  const int tile0 = TWO ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = TWO ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  const uint32_t tiles = smem_u32(smem);
  uint8_t* staging = smem + C::STAGES * C::STAGE_BYTES;  // 1024-byte aligned: the tile area is a multiple of 1024
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::STAGING_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), TWO ? 16 : 8);  // one arrival per epilogue warp (of both CTAs when paired)
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (TWO) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"((uint32_t)C::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"((uint32_t)C::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();  // the peer's barriers are initialised before anything signals them remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // everything above ran in the shadow of the previous kernel; its results are visible from here on

  const int num_m = (p.M + TILE_M - 1) / TILE_M, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK_ELEMS - 1) / BK_ELEMS;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
        const int m_blk = tile / num_n, n_blk = tile % num_n;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t a_dst = tiles + stage * C::STAGE_BYTES;
          if (TWO) {
            // CTA 0's barrier counts the bytes of both CTAs; only CTA 0 arms it.
            if (rank == 0) mbar_expect_tx(full_bar(stage), 2u * (uint32_t)C::STAGE_BYTES);
            tma_load_2d_pair(a_dst, &tmA, full_bar(stage), kb * BK_ELEMS, m_blk * TILE_M + (int)rank * BM);
            tma_load_2d_pair(a_dst + C::A_BYTES, &tmB, full_bar(stage), kb * BK_ELEMS, n_blk * BN + (int)rank * (BN / 2));
          } else {
            mbar_expect_tx(full_bar(stage), (uint32_t)C::STAGE_BYTES);
            tma_load_2d(a_dst, &tmA, full_bar(stage), kb * BK_ELEMS, m_blk * BM);
            tma_load_2d(a_dst + C::A_BYTES, &tmB, full_bar(stage), kb * BK_ELEMS, n_blk * BN);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
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
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc_iter = 0;
      bool ok = true;
      // Descriptors differ only in the start-address field of their low word, so the loop below advances that
      // word with one add per MMA instead of rebuilding 64-bit descriptors (this single thread's instruction
      // stream is what paces the tensor core).
      constexpr uint32_t DESC_HI = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);  // SBO, version, 128-byte swizzle
      const uint32_t a_lo0 = ((tiles & 0x3FFFFu) >> 4) | (1u << 16);
      uint32_t a_lo = a_lo0;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step, ++acc_iter) {
        const int acc = acc_iter & 1;
        const uint32_t acc_phase = (uint32_t)(acc_iter >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        uint32_t accumulate = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          const uint32_t b_lo = a_lo + (uint32_t)(C::A_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK_BYTES / UMMA_K_BYTES; ++k) {
            umma_lo<KIND, TWO>(d_tmem, a_lo + (uint32_t)(k * (UMMA_K_BYTES >> 4)), b_lo + (uint32_t)(k * (UMMA_K_BYTES >> 4)), DESC_HI,
                               IDESC, accumulate);
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
    // Two warps share each TMEM lane quarter and split the tile's 64-column chunks between them, so one warp's
    // TMEM / shared-memory / store latencies are covered by the other warp on the same scheduler.
    const int quad = warp & 3;          // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
    const int half = (warp - 2) >> 2;   // which half of the tile's column chunks this warp takes
    const OutT* bias = static_cast<const OutT*>(p.bias);
    const OutT* residual = static_cast<const OutT*>(p.residual);
    OutT* out = static_cast<OutT*>(p.out);
    const float w_scale = (KIND == KIND_I8) ? *p.w_scale : 1.0f;
    const bool vec_ok = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                        (!bias || (reinterpret_cast<uintptr_t>(bias) & 15) == 0) &&
                        (!residual || ((p.ldr % 8 == 0) && (reinterpret_cast<uintptr_t>(residual) & 15) == 0));
    const bool use_tma = (BN >= 64) && p.tma_store;
    uint8_t* buf = staging + (warp - 2) * 4096;  // this warp's [32 rows x 128 B] staging tile
    int acc_iter = 0;
    // Pulls a tile's residual rows towards L2 ahead of time, so the epilogue's loads do not each pay a DRAM
    // round trip: lane l touches the four 128-byte lines of row l that the tile covers.
    auto prefetch_residual = [&](int t) {
      if (p.epilogue != TTB_EPI_BIAS_RESIDUAL || t >= num_tiles) return;
      const int r = (t / num_n) * TILE_M + (int)rank * BM + quad * 32 + lane, c0 = (t % num_n) * BN;
      if (r >= p.M) return;
      const OutT* rp = residual + (long long)r * p.ldr + c0;
#pragma unroll
      for (int c = 0; c < BN; c += 64)
        if (c0 + c < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + c));
    };
    // Coalesced fetch of a [32 rows x 64 columns] residual block: 8 lanes per 128-byte row, 4 rows per instruction.
    auto load_residual = [&](uint4 (&dst)[8], int rb, int c0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int grow = rb + i * 4 + (lane >> 3), gcol = c0 + (lane & 7) * 8;
        dst[i] = (grow < p.M && gcol < p.N) ? __ldg(reinterpret_cast<const uint4*>(residual + (long long)grow * p.ldr + gcol))
                                            : make_uint4(0, 0, 0, 0);
      }
    };
    prefetch_residual(tile0);
    auto release_accumulator = [&](int a) {  // one arrival per epilogue warp on the MMA-issuing CTA's barrier
      if (TWO && rank != 0) mbar_arrive_remote(tempty_bar(a), 0);
      else mbar_arrive(tempty_bar(a));
    };
    for (int tile = tile0; tile < num_tiles; tile += tile_step, ++acc_iter) {
      const int m_blk = tile / num_n, n_blk = tile % num_n;
      const int acc = acc_iter & 1;
      const uint32_t acc_phase = (uint32_t)(acc_iter >> 1) & 1u;
      const int row_base = m_blk * TILE_M + (int)rank * BM + quad * 32;
      const int row = row_base + lane;
      constexpr int kChunks = (BN >= 64) ? BN / 64 : 1;
      constexpr int kPerWarp = (kChunks >= 2) ? kChunks / 2 : 1;
      // this warp's chunks of the tile: [c_beg, c_end), clipped to the columns that exist
      const int valid_chunks = min(kChunks, (p.N - n_blk * BN + 63) / 64);
      const int c_beg = (kChunks >= 2) ? half * kPerWarp : 0;
      const int c_end = (kChunks >= 2 || half == 0) ? min(c_beg + kPerWarp, valid_chunks) : 0;
      const bool staged_work = use_tma && c_beg < c_end;
      uint4 res[8];
      if (staged_work && p.epilogue == TTB_EPI_BIAS_RESIDUAL) load_residual(res, row_base, n_blk * BN + c_beg * 64);  // before the wait
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) break;
      tc_fence_after();
      prefetch_residual(tile + tile_step);  // the next tile's rows, a whole mainloop ahead
      const float rs = (KIND == KIND_I8 && row < p.M) ? p.row_scale[row] * w_scale : 1.0f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      if (use_tma || half == 1) {
        if (!staged_work) {  // nothing to do for this warp on this tile: just hand the accumulator back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) release_accumulator(acc);
          continue;
        }
        // ---- 64 output columns at a time: TMEM -> registers -> (bias, activation, residual) -> swizzled shared
        //      memory tile -> one TMA store per warp. Residual rows are fetched with coalesced 16-byte loads
        //      (8 lanes per 128-byte row) and handed over through the same tile.
#pragma unroll 1
        for (int cc = c_beg; cc < c_end; ++cc) {
          const int col0 = n_blk * BN + cc * 64;
          if (cc != c_beg && p.epilogue == TTB_EPI_BIAS_RESIDUAL) load_residual(res, row_base, col0);
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
          }
          // two 32-column halves, to keep the live register set small
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int colh = col0 + hh * 32;
            uint4 bq[4];
            if (p.epilogue != TTB_EPI_NONE) {
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8)
                bq[g8] = (colh + g8 * 8 < p.N) ? __ldg(reinterpret_cast<const uint4*>(bias + colh + g8 * 8)) : make_uint4(0, 0, 0, 0);
            }
            uint32_t r0[32];
            tmem_ld32_issue(taddr + (uint32_t)(cc * 64 + hh * 32), r0);
            tmem_ld_wait();
            if (hh == 1 && cc == c_end - 1) {  // this warp's share of the accumulator is in registers: hand it back now
              tc_fence_before();
              __syncwarp();
              if (lane == 0) release_accumulator(acc);
            }
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = (KIND == KIND_I8) ? (float)(int)r0[j] * rs : __uint_as_float(r0[j]);
            if (p.epilogue != TTB_EPI_NONE) {
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                float bb[8];
                unpack8<OutT>(bq[g8], bb);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[g8 * 8 + j] += bb[j];
              }
            }
            if (p.epilogue == TTB_EPI_BIAS_GELU) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {  // 0.5x(1 + tanh(0.79788456(x + 0.044715x^3))), regrouped to six operations
                const float x = v[j], hx = 0.5f * x;
                const float t = tanh_fast(x * fmaf(x * x, 0.7978845608028654f * 0.044715f, 0.7978845608028654f));
                v[j] = fmaf(hx, t, hx);
              }
            } else if (p.epilogue == TTB_EPI_BIAS_TANH) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = tanh_fast(v[j]);
            } else if (p.epilogue == TTB_EPI_BIAS_RESIDUAL) {
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                float q[8];
                unpack8<OutT>(*reinterpret_cast<const uint4*>(buf + lane * 128 + (((hh * 4 + g8) ^ (lane & 7)) << 4)), q);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[g8 * 8 + j] += q[j];
              }
            }
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8)
              *reinterpret_cast<uint4*>(buf + lane * 128 + (((hh * 4 + g8) ^ (lane & 7)) << 4)) = pack8<OutT>(&v[g8 * 8]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmO, smem_u32(buf), col0, row_base);
            bulk_commit();
          }
        }
        continue;
      }
      // ---- direct path (narrow tiles or unaligned output): the first warp of each lane quarter walks the tile
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), r);
        const int col0 = n_blk * BN + c * 32;
        if (row >= p.M || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (KIND == KIND_I8) ? (float)(int)r[j] * rs : __uint_as_float(r[j]);
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
          for (int j = 0; j < 32; ++j) {
            const float x = v[j];
            v[j] = x * 0.5f * (1.0f + tanh_fast(0.7978845608028654f * (x + 0.044715f * x * x * x)));
          }
        } else if (p.epilogue == TTB_EPI_BIAS_TANH) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = tanh_fast(v[j]);
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
        OutT* op = out + (long long)row * p.ldo + col0;
        if (full) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            Vec8<OutT> o;
#pragma unroll
            for (int j = 0; j < 8; ++j) o.v[j] = v[i * 8 + j];
            o.store(op + i * 8);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) op[j] = from_f<OutT>(v[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release_accumulator(acc);
    }
    // every TMA store issued by this warp must be complete before its shared memory goes away
    if (use_tma && lane == 0) bulk_wait<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------------ teardown (all roles reach this)
  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    if (TWO) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, (int)TTB_ERR_DEVICE_WAIT);
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// 2-D row-major matrix [rows, k] with `ld` elements between rows; box = [box_rows, 128 bytes of k], 128-byte swizzle.
// Used for both operands (K-major tiles) and for the output (32-row x 64-column store boxes).
int make_map(ttb_ctx* ctx, CUtensorMap* map, int kind, const void* ptr, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(ctx, TTB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const int es = (kind == KIND_I8) ? 1 : 2;
  const CUtensorMapDataType dt = kind == KIND_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                 : (kind == KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * es};
  cuuint32_t box[2] = {(cuuint32_t)(BK_BYTES / es), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ctx, TTB_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (rows=%lld k=%lld ld=%lld)", (int)r,
                                     (long long)rows, (long long)k, (long long)ld);
  return TTB_OK;
}

template <int BN, int KIND, typename OutT, bool TWO>
int launch_tc(ttb_ctx* ctx, const void* A, int64_t lda, const void* W, const GemmParams& p) {
  using C = Cfg<BN, TWO>;
  constexpr int TILE_M = TWO ? 2 * BM : BM;
  CUtensorMap tmA, tmB;
  int s = make_map(ctx, &tmA, KIND, A, p.M, p.K, lda, BM);
  if (s) return s;
  s = make_map(ctx, &tmB, KIND, W, p.N, p.K, p.K, TWO ? BN / 2 : BN);
  if (s) return s;
  GemmParams q = p;
  CUtensorMap tmO = tmA;  // placeholder when the direct-store epilogue is used
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.bias) |
                           reinterpret_cast<uintptr_t>(p.residual)) & 15) == 0;
  // The staged epilogue reads bias and residual eight columns at a time, and a TMA store clips a row at 16-byte
  // granularity: with a ragged N it writes zeros into the columns up to the next multiple of 8. So a ragged N takes
  // this route only without bias/residual and when the caller declared those columns scratch (p.tma_store on entry).
  q.tma_store = (BN >= 64 && aligned16 && p.ldo % 8 == 0 && (p.N % 8 == 0 || (p.epilogue == TTB_EPI_NONE && p.tma_store)) &&
                 (!p.residual || p.ldr % 8 == 0)) ? 1 : 0;
  if (q.tma_store) {
    const int out_kind = std::is_same<OutT, __nv_bfloat16>::value ? KIND_BF16 : KIND_F16;
    s = make_map(ctx, &tmO, out_kind, p.out, p.M, p.N, p.ldo, 32);
    if (s) return s;
  }
  auto kern = gemm_tc_kernel<BN, KIND, OutT, TWO>;
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
  if (!TWO) {
    const int grid = (int)(num_tiles < ctx->sm_count ? num_tiles : ctx->sm_count);
    cudaError_t e = launch_pdl(kern, dim3((unsigned)grid), dim3(kThreads), C::SMEM_BYTES, ctx->stream, tmA, tmB, tmO, q);
    if (e != cudaSuccess) return fail(ctx, TTB_ERR_CUDA, "launch of gemm_tc failed: %s", cudaGetErrorString(e));
    return launched(ctx, "gemm_tc");
  }
  const int clusters = (int)(num_tiles < max_clusters[dev] ? num_tiles : max_clusters[dev]);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (unsigned)clusters);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmO, q);
  if (e != cudaSuccess) return fail(ctx, TTB_ERR_CUDA, "cluster launch of gemm_tc failed: %s", cudaGetErrorString(e));
  return launched(ctx, "gemm_tc_pair");
}

// TTB_GEMM_PAIR: 0 disables the two-CTA variant, 2 uses it for every shape with at least half a wave of pair tiles
// (measurement switches); unset = chosen by shape.
int pair_mode() {
  static const int mode = [] {
    const char* e = getenv("TTB_GEMM_PAIR");
    return (e && e[0] == '0') ? 0 : ((e && e[0] == '2') ? 2 : 1);
  }();
  return mode;
}

template <int KIND, typename OutT>
int pick_tile(ttb_ctx* ctx, const void* A, int64_t lda, const void* W, const GemmParams& p) {
  // Large problems: CTA pairs on 256 x 256 tiles (less L2->SM traffic per flop). Otherwise the largest single-CTA
  // N-tile that still gives every SM a tile; small problems use narrow tiles to spread over SMs.
  const int64_t num_m = (p.M + BM - 1) / BM;
  auto tiles = [&](int bn) { return num_m * ((p.N + bn - 1) / bn); };
  const int64_t pair_tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * (int64_t)((p.N + 255) / 256);
  // Measured on B200 in back-to-back launches at M = 18424 (single CTA -> pair, TFLOP/s): N=2304 K=768 1097 -> 1228,
  // N=3072 K=768 1088 -> 1165, N=768 K=3072 1171 -> 1273, but N=768 K=768 789 -> 756: pairs win unless both the
  // mainloop and the row of tiles are short.
  const int64_t k_bytes = (int64_t)p.K * (KIND == KIND_I8 ? 1 : 2);
  const bool pair_pays = k_bytes >= 4096 || p.N >= 1536;
  if (pair_mode() && pair_tiles >= ctx->sm_count / 2 && (pair_pays || pair_mode() == 2)) return launch_tc<256, KIND, OutT, true>(ctx, A, lda, W, p);
  if (tiles(256) >= ctx->sm_count) return launch_tc<256, KIND, OutT, false>(ctx, A, lda, W, p);
  if (tiles(128) >= ctx->sm_count) return launch_tc<128, KIND, OutT, false>(ctx, A, lda, W, p);
  if (tiles(64) >= ctx->sm_count / 2) return launch_tc<64, KIND, OutT, false>(ctx, A, lda, W, p);
  return launch_tc<32, KIND, OutT, false>(ctx, A, lda, W, p);
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

}  // namespace

// =================================================================================================
extern "C" int ttb_linear(ttb_ctx* ctx, int dtype, const void* A, int64_t lda, const void* Wp, const void* bias,
                          const void* residual, int64_t ldr, int64_t M, int64_t N, int64_t K, int epilogue, void* out,
                          int64_t ldo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, dtype == TTB_F16 || dtype == TTB_BF16, "linear: dtype must be F16 or BF16 (use ttb_matmul for F32)");
  const int pad_scratch = (epilogue & TTB_EPI_FLAG_ROW_PADDING_IS_SCRATCH) ? 1 : 0;
  epilogue &= ~TTB_EPI_FLAG_ROW_PADDING_IS_SCRATCH;
  int s = check_linear(ctx, "linear", A, Wp, bias, residual, M, N, K, epilogue, out, ldo, 8);
  if (s || M == 0) return s;
  TTB_REQUIRE(ctx, lda >= K && lda % 8 == 0, "linear: lda must be >= K and a multiple of 8");
  DeviceGuard g(ctx->device);
  GemmParams p{(int)M, (int)N, (int)K, out, ldo, bias, residual, ldr, nullptr, nullptr, epilogue, pad_scratch, ctx->d_status};
  if (dtype == TTB_F16) return pick_tile<KIND_F16, __half>(ctx, A, lda, Wp, p);
  return pick_tile<KIND_BF16, __nv_bfloat16>(ctx, A, lda, Wp, p);
}

extern "C" int ttb_linear_int8(ttb_ctx* ctx, int out_dtype, const int8_t* Aq, const float* row_scale, const int8_t* Wq,
                               const float* w_scale, const void* bias, const void* residual, int64_t ldr, int64_t M,
                               int64_t N, int64_t K, int epilogue, void* out, int64_t ldo) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, out_dtype == TTB_F16 || out_dtype == TTB_BF16, "linear_int8: output dtype must be F16 or BF16");
  int s = check_linear(ctx, "linear_int8", Aq, Wq, bias, residual, M, N, K, epilogue, out, ldo, 16);
  if (s || M == 0) return s;
  TTB_REQUIRE(ctx, row_scale && w_scale, "linear_int8: null scale pointer");
  DeviceGuard g(ctx->device);
  GemmParams p{(int)M, (int)N, (int)K, out, ldo, bias, residual, ldr, row_scale, w_scale, epilogue, 0, ctx->d_status};
  if (out_dtype == TTB_F16) return pick_tile<KIND_I8, __half>(ctx, Aq, K, Wq, p);
  return pick_tile<KIND_I8, __nv_bfloat16>(ctx, Aq, K, Wq, p);
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
