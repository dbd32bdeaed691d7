// Self-attention over packed variable-length batches on the 5th-generation tensor cores.
//
// Persistent kernel, one CTA per SM, two independent streams per CTA. A work item is one 128-row query tile of one
// (sequence, head); a stream walks the key/value tiles (128 rows) of one item after the other as one flat sequence of
// tiles g = 0, 1, 2, ...
//   warps 0, 2  : TMA loaders of stream 0 / 1 - the item's Q tile (double-buffered) and K_g / V_g into 2-stage rings, by
//                 two independent cursors (Q + K tiles, V tiles) that each issue as soon as their slot is free, so the next
//                 item's Q and first K tile are in flight a whole tile before they are needed.
//                 Every tile is a [128 rows x 64 columns] 128-byte-swizzled box straight out of the [T, 3H] QKV matrix.
//   warps 1, 3  : MMA issuers of stream 0 / 1 - S = Q K_g^T (128x128x64, fp32 in TMEM) and O += P V_g (128x64x128) with P
//                 read from TMEM and V used in place as an MN-major operand. Per stream the order is
//                 QK(0) | QK(g+1) PV(g) | ..., across item boundaries: QK(g+1) goes out as soon as the softmax warps hold
//                 the scores of tile g in registers, so the next scores are in TMEM before the current softmax ends. A
//                 wait in an issuing thread only returns once the MMAs that thread has issued have drained, so each
//                 stream has its own issuer. It waits for the softmax warps' go-ahead first (which lets its earlier MMAs
//                 drain) and then for the operand tiles of the group (a barrier poll each): the softmax warps never wait
//                 on a load. Measured with per-phase cycle stamps on 37 x 512: a stream's tile period is the softmax
//                 warps' serial chain (score load 160-200 cycles, 128 exponentials per thread with their sums and packing
//                 2650-2900 while the other stream's warp shares the scheduler, P store 115-160, two satisfied barrier
//                 waits 110-260 each), plus per item the output pass and 600-1300 cycles of bookkeeping.
//   warps 4..7  : softmax of stream 0, warps 8..11: of stream 1 (registers are moved from the first
//                 warpgroup to the softmax ones with setmaxnreg) - one query row per thread: scores from TMEM, running
//                 max / sum in fp32, exp2 with the scale folded in, P written back to TMEM as packed 16-bit pairs.
//                 O accumulates in TMEM across key tiles. The row maximum is taken on an item's first tile only; later
//                 tiles reuse it and fall back to a rescale of O only if a probability would leave the 16-bit range
//                 (row sum above 2^15), which real score distributions do not reach. The final division by the running
//                 sum makes the result independent of the reference maximum. With a mask operand (one row of keys per
//                 sequence) a warp fetches the tile's 128 entries once and, if any is set, adds them where the scores
//                 leave TMEM. An item's output (O / l) leaves through the item's own Q buffer as whole 128-byte rows.
// TMEM (all 512 columns): S0 | S1 (128 each) | O0 | O1 (64 each) | P0 | P1 (64 each).
// Items are ordered longest sequence first; a stream's first item is fixed, every further one is the next item nobody has
// taken (a counter in global memory, fetched one item ahead by the stream's loader), so the streams finish together even
// when their items differ in length or their SMs in speed (with a fixed round-robin deal the slowest CTA of the ragged
// benchmark batch finished 10.5 us after the median one, of 77).
// Every wait is bounded; on expiry the CTA raises a flag, frees its TMEM and the host sees TTB_ERR_DEVICE_WAIT.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "ttb_common.cuh"
#include "ttb_sm100.cuh"

using namespace ttb;
using namespace ttb::sm100;

namespace {

constexpr int QT = 128, KT = 128, D = 64;
constexpr int kMaxB = 512;       // sequences per launch that the in-kernel schedule tables hold
constexpr int kSortMaxB = 256;   // above this the (quadratic) length ranking is skipped and sequences keep their order
constexpr int kThreads = 384;    // three warpgroups: {loader 0, MMA 0, loader 1, MMA 1}, softmax stream 0, softmax stream 1
constexpr int TILE_BYTES = 128 * 128;  // a [128 rows x 128 B] tile
// per stream: Q[2], K[2], V[2]
constexpr int SMEM_STREAM = 6 * TILE_BYTES;
constexpr int SMEM_CU = 2 * SMEM_STREAM;                   // int[kMaxB + 1] token offsets
constexpr int SMEM_PREFIX = SMEM_CU + (kMaxB + 1) * 4;     // int[kMaxB + 1] items before each ranked sequence
constexpr int SMEM_ORDER = SMEM_PREFIX + (kMaxB + 1) * 4;  // uint16[kMaxB] sequence at each rank
constexpr int SMEM_BARS = (SMEM_ORDER + kMaxB * 2 + 63) / 64 * 64;
constexpr int kBarsPerStream = 16;
constexpr int kRing = 8;  // item ids a stream's loader has published and the other roles may still read
constexpr int kRingInts = 8;  // per published item: id, tok0, len, q0, head, key tiles
constexpr int SMEM_MISC = 2 * kBarsPerStream * 8 + 64 + 2 * kRing * kRingInts * 4;  // barriers, TMEM slot, flags, item rings
constexpr int SMEM_MASKROW = (SMEM_BARS + SMEM_MISC + 15) / 16 * 16;                // float[8 softmax warps][128]: a tile's mask entries
constexpr int SMEM_BYTES = SMEM_MASKROW + 8 * 128 * 4;
constexpr uint32_t TMEM_COLS = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRowSumLimit = 32768.0f;  // a tile row sum below this keeps every probability inside fp16 / bf16 range

struct Params {
  void* out;
  const int32_t* cu;
  int batch, heads, causal;
  float scale;
  int* status;
  int* sched;  // [0] items handed out beyond every stream's first, [1] CTAs that have finished; both zero between launches
  int staged;  // measurement switch: 0 = output rows stored straight from registers
  const float* mask;      // MASK kernels: additive fp32 mask, one row of keys per sequence: mask[b * mask_bs + key]
  long long mask_bs;
};

struct Item {
  int tok0, len, q0, head;
  int n;    // key tiles this query tile visits
  int seq;  // which sequence of the batch
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

// Item `i` of the launch: rank-ordered (sequence, 128-row query tile) x head.
__device__ __forceinline__ Item decode_item(int i, const Params& p, const int* s_cu, const int* s_prefix, const uint16_t* s_order) {
  Item it;
  it.head = i % p.heads;
  const int pidx = i / p.heads;
  int lo = 0, hi = p.batch;  // largest r with s_prefix[r] <= pidx
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_prefix[mid] <= pidx) lo = mid;
    else hi = mid;
  }
  const int seq = s_order[lo];
  it.seq = seq;
  it.tok0 = s_cu[seq];
  it.len = s_cu[seq + 1] - it.tok0;
  const int qt = pidx - s_prefix[lo];
  it.q0 = qt * QT;
  const int n_all = (it.len + KT - 1) / KT;
  it.n = p.causal ? min(n_all, qt + 1) : n_all;
  return it;
}

// Where one side (score MMAs or output MMAs) of a stream stands in the stream's flat tile sequence.
struct Cursor {
  int i;        // item, >= n_items when the stream is exhausted
  int j, n;     // tile within the item, tiles of the item
  uint32_t g;   // tiles before this one in the stream
  uint32_t nq;  // items before this one in the stream
};

template <typename T, bool MASK>
__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tm, const Params p) {
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_S = idesc_f16(FMT, 128, KT, 0);  // Q (K-major) x K^T (K-major)
  constexpr uint32_t IDESC_O = idesc_f16(FMT, 128, D, 1);   // P (TMEM) x V (MN-major)

  extern __shared__ __align__(1024) uint8_t smem[];  // the swizzled tiles need 1024-byte alignment
  const uint32_t base = smem_u32(smem);
  if (base & 1023u) {  // cannot happen with the alignment above; refuse rather than compute garbage
    pdl_wait();
    if (threadIdx.x == 0) atomicExch(p.status, (int)TTB_ERR_DEVICE_WAIT);
    return;
  }
  int* s_cu = reinterpret_cast<int*>(smem + SMEM_CU);
  int* s_prefix = reinterpret_cast<int*>(smem + SMEM_PREFIX);
  uint16_t* s_order = reinterpret_cast<uint16_t*>(smem + SMEM_ORDER);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BARS);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int s, int k) { return bar0 + 8u * (s * kBarsPerStream + k); };
  auto q_full = [&](int s, int b) { return bar(s, b); };
  auto q_empty = [&](int s, int b) { return bar(s, 2 + b); };
  auto k_full = [&](int s, int st) { return bar(s, 4 + st); };
  auto k_empty = [&](int s, int st) { return bar(s, 6 + st); };
  auto v_full = [&](int s, int st) { return bar(s, 8 + st); };
  auto v_empty = [&](int s, int st) { return bar(s, 10 + st); };
  auto s_full = [&](int s) { return bar(s, 12); };
  auto s_free = [&](int s) { return bar(s, 13); };
  auto p_ready = [&](int s) { return bar(s, 14); };
  auto o_done = [&](int s) { return bar(s, 15); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kBarsPerStream);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // Work distribution: a stream's first item is fixed (2 * blockIdx.x + stream); every further one is the next item nobody
  // has taken yet, fetched by the stream's loader from a counter in global memory and published here for the stream's
  // other roles. Items are ranked longest first, so whichever stream is free takes the longest remaining one.
  volatile int* s_produced = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]: items published so far
  volatile int* s_ring = reinterpret_cast<volatile int*>(tmem_slot + 4);      // [2][kRing][kRingInts]: id (n_items = no more work) and decoded form
  auto smem_q = [&](int s, int b) { return base + (uint32_t)(s * SMEM_STREAM + b * TILE_BYTES); };
  auto smem_k = [&](int s, int st) { return base + (uint32_t)(s * SMEM_STREAM + (2 + st) * TILE_BYTES); };
  auto smem_v = [&](int s, int st) { return base + (uint32_t)(s * SMEM_STREAM + (4 + st) * TILE_BYTES); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = p.heads * D;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      for (int k = 0; k < 13; ++k) mbar_init(bar(s, k), 1);  // TMA and MMA-commit barriers
      // a Q buffer is free again once the item's last score MMA has read it and the four softmax warps have used it as
      // the staging tile of the item's output (see flush_output)
      mbar_init(q_empty(s, 0), 5);
      mbar_init(q_empty(s, 1), 5);
      mbar_init(s_free(s), 4);                                // one arrival per softmax warp
      mbar_init(p_ready(s), 4);
      mbar_init(o_done(s), 1);
    }
    *abort_flag = 0;
    s_produced[0] = 0;
    s_produced[1] = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  if (threadIdx.x == 64) prefetch_tensormap(&tm);  // a kernel parameter: fetching it does not depend on the previous kernel
  pdl_wait();  // everything above ran in the shadow of the previous kernel; global memory is touched from here on
  // ---- schedule tables (every CTA builds the same ones) -----------------------------------------------------------
  for (int i = threadIdx.x; i <= p.batch; i += kThreads) s_cu[i] = p.cu[i];
  __syncthreads();
  // rank sequences by descending key-tile count (ties by index): the rank is the position in the item order
  for (int i = threadIdx.x; i < p.batch; i += kThreads) {
    int rank = i;
    if (p.batch <= kSortMaxB) {
      const int mine = (s_cu[i + 1] - s_cu[i] + KT - 1) / KT;
      rank = 0;
      for (int j = 0; j < p.batch; ++j) {
        const int other = (s_cu[j + 1] - s_cu[j] + KT - 1) / KT;
        rank += (other > mine || (other == mine && j < i)) ? 1 : 0;
      }
    }
    s_order[rank] = (uint16_t)i;
  }
  __syncthreads();
  if (warp == 0) {  // exclusive scan of the query-tile counts in rank order
    int carry = 0;
    for (int r0 = 0; r0 < p.batch; r0 += 32) {
      const int r = r0 + lane;
      int tiles = 0;
      if (r < p.batch) {
        const int seq = s_order[r];
        tiles = (s_cu[seq + 1] - s_cu[seq] + QT - 1) / QT;
      }
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (r < p.batch) s_prefix[r] = carry + incl - tiles;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_prefix[p.batch] = carry;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_items = s_prefix[p.batch] * p.heads;
  // the id of a stream's nq-th item, once its loader has published it (bounded wait; n_items when giving up)
  auto item_at = [&](int s, uint32_t nq) -> int {
    if (s_produced[s] <= (int)nq) {
      const long long t0 = clock64();
      while (s_produced[s] <= (int)nq) {
        if (*abort_flag || clock64() - t0 > kWaitCycles) {
          *abort_flag = 1;
          return n_items;
        }
      }
    }
    return s_ring[(s * kRing + (int)(nq & (kRing - 1))) * kRingInts];
  };
  // the decoded form of a published item (decoded once, by the loader)
  auto item_read = [&](int s, uint32_t nq) -> Item {
    const volatile int* e = s_ring + (s * kRing + (int)(nq & (kRing - 1))) * kRingInts;
    Item it;
    it.tok0 = e[1];
    it.len = e[2];
    it.q0 = e[3];
    it.head = e[4];
    it.n = e[5];
    it.seq = e[6];
    return it;
  };
  auto tmem_s = [&](int s) { return tmem + (uint32_t)(s * 128); };
  auto tmem_o = [&](int s) { return tmem + (uint32_t)(256 + s * 64); };
  auto tmem_p = [&](int s) { return tmem + (uint32_t)(384 + s * 64); };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0 || warp == 2) {
      // ------------------------------------------------------------------ loader of stream `s`
      const int s = warp >> 1;
      if (lane == 0) {
        // Two cursors walk the stream's tile sequence independently: one issues Q and K tiles, the other V tiles, each
        // as soon as its ring slot is free. (Were they one in-order sequence, the next item's Q and first K tile would
        // queue behind the current item's last V tile, whose slot frees late, and arrive a tile too late.) Nothing
        // blocks: slots are polled, and the thread gives up when neither cursor has moved for the wait limit.
        struct LoadCursor {
          int i, j, n;
          uint32_t g, nq;
          Item it;
        } kc, vc;
        int produced = 0, last_id = 0;
        auto produce = [&]() {  // publishes the id of the stream's next item
          int id = n_items;
          if (produced == 0) id = min(2 * (int)blockIdx.x + s, n_items);
          else if (last_id < n_items) id = min(2 * (int)gridDim.x + atomicAdd(p.sched, 1), n_items);
          last_id = id;
          volatile int* e = s_ring + (s * kRing + (produced & (kRing - 1))) * kRingInts;
          e[0] = id;
          if (id < n_items) {
            const Item it = decode_item(id, p, s_cu, s_prefix, s_order);
            e[1] = it.tok0;
            e[2] = it.len;
            e[3] = it.q0;
            e[4] = it.head;
            e[5] = it.n;
            e[6] = it.seq;
          }
          __threadfence_block();
          s_produced[s] = ++produced;
        };
        produce();
        produce();  // one item ahead of the cursors, so that the counter's round trip is off their path
        kc.i = 2 * (int)blockIdx.x + s;
        kc.j = 0;
        kc.g = 0;
        kc.nq = 0;
        kc.n = 0;
        if (kc.i < n_items) {
          kc.it = item_read(s, 0);
          kc.n = kc.it.n;
        }
        vc = kc;
        bool q_issued = false;
        auto advance = [&](LoadCursor& c) {
          ++c.g;
          if (++c.j == c.n) {
            c.j = 0;
            ++c.nq;
            if ((int)c.nq + 1 >= produced) produce();  // the key cursor leads: it finds item nq published and publishes nq + 1
            c.i = s_ring[(s * kRing + (int)(c.nq & (kRing - 1))) * kRingInts];
            if (c.i < n_items) {
              c.it = item_read(s, c.nq);
              c.n = c.it.n;
            }
          }
        };
        long long t_progress = clock64();
        while (kc.i < n_items || vc.i < n_items) {
          bool progressed = false;
          if (kc.i < n_items) {
            if (kc.j == 0 && !q_issued) {
              const int b = kc.nq & 1;
              if (mbar_test_wait(q_empty(s, b), ((kc.nq >> 1) & 1u) ^ 1u)) {
                mbar_expect_tx(q_full(s, b), TILE_BYTES);
                tma_load_2d(smem_q(s, b), &tm, q_full(s, b), kc.it.head * D, kc.it.tok0 + kc.it.q0);
                q_issued = true;
                progressed = true;
              }
            }
            if (kc.j > 0 || q_issued) {
              const int st = kc.g & 1;
              if (mbar_test_wait(k_empty(s, st), ((kc.g >> 1) & 1u) ^ 1u)) {
                mbar_expect_tx(k_full(s, st), TILE_BYTES);
                tma_load_2d(smem_k(s, st), &tm, k_full(s, st), H + kc.it.head * D, kc.it.tok0 + kc.j * KT);
                advance(kc);
                if (kc.j == 0) q_issued = false;
                progressed = true;
              }
            }
          }
          if (vc.i < n_items) {
            const int st = vc.g & 1;
            if (mbar_test_wait(v_empty(s, st), ((vc.g >> 1) & 1u) ^ 1u)) {
              mbar_expect_tx(v_full(s, st), TILE_BYTES);
              tma_load_2d(smem_v(s, st), &tm, v_full(s, st), 2 * H + vc.it.head * D, vc.it.tok0 + vc.j * KT);
              advance(vc);
              progressed = true;
            }
          }
          if (progressed) {
            t_progress = clock64();
          } else {
            if (*abort_flag) break;
            if (clock64() - t_progress > kWaitCycles) {
              *abort_flag = 1;
              break;
            }
            __nanosleep(400);
          }
        }
        if (*abort_flag) {  // let copies in flight land before shared memory is released
          const long long t0 = clock64();
          while (clock64() - t0 < 4000000LL) {
          }
        }
      }
      __syncwarp();
    } else {
      // ------------------------------------------------------------------ MMA issuer of stream `s` (warp 1: 0, warp 3: 1)
      const int s = warp >> 1;
      if (lane == 0) {
        bool ok = true;
        Cursor qc, pc;  // score side and output side
        auto advance = [&](Cursor& c) {
          ++c.g;
          if (++c.j == c.n) {
            c.j = 0;
            ++c.nq;
            c.i = item_at(s, c.nq);
            c.n = (c.i < n_items) ? item_read(s, c.nq).n : 0;
          }
        };
        qc.j = 0;
        qc.g = 0;
        qc.nq = 0;
        qc.i = item_at(s, 0);
        qc.n = (qc.i < n_items) ? item_read(s, 0).n : 0;
        pc = qc;
        // S = Q K_g^T. Q and K_g are in shared memory and S is free when this is called.
        auto qk = [&]() {
          const int st = qc.g & 1, qb = qc.nq & 1;
          const uint32_t q_lo = desc_lo(smem_q(s, qb)), k_lo = desc_lo(smem_k(s, st));
#pragma unroll
          for (int k = 0; k < D / 16; ++k) umma_f16(tmem_s(s), q_lo + k * 2, k_lo + k * 2, IDESC_S, k != 0);  // 32 bytes of d per step
          tc_commit(s_full(s));
          tc_commit(k_empty(s, st));
          if (qc.j == qc.n - 1) tc_commit(q_empty(s, qb));  // last reader of this item's Q
          advance(qc);
        };
        // The operand tiles of a group are waited for here, right before the group is issued and after the wait on
        // the softmax warps (which has already let the MMAs issued before it drain, so these cost a barrier poll each).
        auto operands_of_qk = [&]() {
          bool landed = mbar_wait(k_full(s, qc.g & 1), (qc.g >> 1) & 1u, abort_flag);
          if (landed && qc.j == 0) landed = mbar_wait(q_full(s, qc.nq & 1), (qc.nq >> 1) & 1u, abort_flag);
          return landed;
        };
        if (qc.i < n_items) {
          ok = operands_of_qk();
          if (ok) qk();
        }
        while (ok && pc.i < n_items) {
          // scores of the next tile, once the softmax warps hold the current tile's scores in registers (they also vouch
          // for the Q and K tiles the MMA reads)
          if (qc.i < n_items) {
            if (!mbar_wait(s_free(s), (qc.g - 1) & 1u, abort_flag)) break;
            if (!operands_of_qk()) break;
            tc_fence_after();
            qk();
          }
          // O (+)= P V_g once the softmax warps have released P (and vouched for V_g)
          if (!mbar_wait(p_ready(s), pc.g & 1u, abort_flag)) break;
          if (!mbar_wait(v_full(s, pc.g & 1), (pc.g >> 1) & 1u, abort_flag)) break;
          tc_fence_after();
          const int st = pc.g & 1;
          const uint32_t v_lo = desc_lo(smem_v(s, st));
#pragma unroll
          for (int k = 0; k < KT / 16; ++k)  // 16 keys per MMA: 8 TMEM columns of P, 16 rows (of 128 bytes) of V
            umma_f16_ts(tmem_o(s), tmem_p(s) + (uint32_t)(k * 8), v_lo + (uint32_t)(k * (16 * 128 >> 4)), IDESC_O, (pc.j | k) != 0);
          tc_commit(o_done(s));
          tc_commit(v_empty(s, st));
          advance(pc);
        }
      }
      __syncwarp();
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ------------------------------------------------------------------ softmax + output (one query row per thread)
    const int s = (warp - 4) >> 2;
    const int quad = warp & 3;                  // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may touch
    const int row = quad * 32 + lane;           // row within the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t ts = tmem_s(s) + lane_addr, to = tmem_o(s) + lane_addr, tp = tmem_p(s) + lane_addr;
    // With a mask, the scores of a tile whose mask entries are not all zero are moved to the exponent's domain where they are
    // loaded (s * scale * log2 e + mask * log2 e), and everything after that works with a scale of one for that tile.
    const float sc_plain = p.scale * kLog2e;
    uint32_t g = 0, nq = 0;
    bool ok = true;
    // The output pass of an item (O / l to global memory) is deferred to the start of the stream's next item, before that
    // item's first scores are loaded (so that they do not hold the registers meanwhile): the last output MMA has 200 - 300
    // cycles left to run at that point, and the next item's first scores are being computed.
    bool pend = false;
    float pend_inv = 0.f;
    T* pend_base = nullptr;  // first output element of this warp's 32 rows of the pending item
    int pend_rows = 0;       // how many of those rows exist in the sequence
    int pend_qb = 0;         // the pending item's Q buffer
    // Output pass: O / l of the warp's 32 rows goes through shared memory, so that the global stores are whole 128-byte
    // rows (one lane per row straight from registers costs 32 cache lines per store instruction, and with four warps
    // flushing at once that was 2000 - 3000 cycles per item). The staging tile is the item's own Q buffer: its last
    // reader, the item's last score MMA, completed before the scores of that tile were loaded.
    auto flush_output = [&]() {  // whole warp; g = tiles finished so far, the pending item's last tile is g - 1
      if (!__all_sync(0xffffffffu, mbar_wait(o_done(s), (g - 1) & 1u, abort_flag))) return false;
      tc_fence_after();
      uint8_t* stage = smem + s * SMEM_STREAM + pend_qb * TILE_BYTES + quad * 32 * 128;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32_issue(to + (uint32_t)(c * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          uint4 q;
          q.x = pack2<T>(__uint_as_float(r[g8 * 8 + 0]) * pend_inv, __uint_as_float(r[g8 * 8 + 1]) * pend_inv);
          q.y = pack2<T>(__uint_as_float(r[g8 * 8 + 2]) * pend_inv, __uint_as_float(r[g8 * 8 + 3]) * pend_inv);
          q.z = pack2<T>(__uint_as_float(r[g8 * 8 + 4]) * pend_inv, __uint_as_float(r[g8 * 8 + 5]) * pend_inv);
          q.w = pack2<T>(__uint_as_float(r[g8 * 8 + 6]) * pend_inv, __uint_as_float(r[g8 * 8 + 7]) * pend_inv);
          if (p.staged) *reinterpret_cast<uint4*>(stage + lane * 128 + (((c * 4 + g8) ^ (lane & 7)) << 4)) = q;  // swizzled: no bank conflicts either way
          else if (lane < pend_rows) *reinterpret_cast<uint4*>(pend_base + (long long)lane * H + (c * 4 + g8) * 8) = q;
        }
      }
      __syncwarp();
      if (p.staged) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // four rows of 128 bytes per instruction
          const int r = k * 4 + (lane >> 3), j = lane & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 128 + ((j ^ (r & 7)) << 4));
          if (r < pend_rows) *reinterpret_cast<uint4*>(pend_base + (long long)r * H + j * 8) = v;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(q_empty(s, pend_qb));
      pend = false;
      return true;
    };

    for (int i = item_at(s, 0); i < n_items && ok; ++nq, i = item_at(s, nq)) {
      const Item it = item_read(s, nq);
      const int qrow = it.q0 + row;  // row within the sequence
      float m_used = -INFINITY, l_run = 0.f;

      for (int j = 0; j < it.n; ++j, ++g) {
        const int k0 = j * KT;
        // The previous item's output pass, before this tile's scores occupy the registers. It reads O before this warp's
        // next p_ready arrival, which is what the next output MMA (the one that overwrites O) waits for; it also proves
        // PV(g-1) complete, so P may be rewritten.
        if (pend && !flush_output()) { ok = false; break; }
        if (!__all_sync(0xffffffffu, mbar_wait(s_full(s), g & 1u, abort_flag))) { ok = false; break; }  // warp-uniform
        tc_fence_after();
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32_issue(ts + (uint32_t)(c * 32), sr[c]);
        tmem_ld_wait();
        tc_fence_before();  // S_g is in registers: the next scores may overwrite it (one phase per tile)
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free(s));
        float sc = sc_plain;
        bool tile_dead = false;  // MASK: every key of the tile is masked out for every row of this warp
        if (MASK) {
          const float* mrow = p.mask + (long long)it.seq * p.mask_bs + k0;
          const float sc_in = sc_plain;
          const int valid = it.len - k0;  // keys of the tile that exist; the others are set to -inf below
          // The warp fetches the tile's 128 entries once, four per lane, coalesced (any row pitch and alignment). A padding
          // mask is zero over most tiles: when none of the entries is set the scores are left alone. Otherwise the entries go
          // through a 512-byte row of shared memory, from which every thread reads all of them 16 bytes at a time.
          float mine[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) mine[u] = (u * 32 + lane < valid) ? __ldg(mrow + u * 32 + lane) : 0.f;
          // A tile whose entries are all at a padding mask's -10000 contributes exact zeros once the row has seen a key
          // that is not masked (its maximum is then thousands of octaves above anything in this tile): no arithmetic.
          const bool all_off = __all_sync(0xffffffffu, (lane >= valid || mine[0] <= -5000.f) && (32 + lane >= valid || mine[1] <= -5000.f) &&
                                                           (64 + lane >= valid || mine[2] <= -5000.f) && (96 + lane >= valid || mine[3] <= -5000.f));
          tile_dead = all_off && j > 0 && __all_sync(0xffffffffu, m_used > -2000.f);
          if (!tile_dead && __any_sync(0xffffffffu, mine[0] != 0.f || mine[1] != 0.f || mine[2] != 0.f || mine[3] != 0.f)) {
            sc = 1.0f;
            float* mtile = reinterpret_cast<float*>(smem + SMEM_MASKROW) + (warp - 4) * 128;
            __syncwarp();  // the previous tile's reads of the row are done
#pragma unroll
            for (int u = 0; u < 4; ++u) mtile[u * 32 + lane] = mine[u] * kLog2e;
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int e = 0; e < 32; e += 4) {
                const float4 mk = *reinterpret_cast<const float4*>(mtile + c * 32 + e);
                sr[c][e] = __float_as_uint(fmaf(__uint_as_float(sr[c][e]), sc_in, mk.x));
                sr[c][e + 1] = __float_as_uint(fmaf(__uint_as_float(sr[c][e + 1]), sc_in, mk.y));
                sr[c][e + 2] = __float_as_uint(fmaf(__uint_as_float(sr[c][e + 2]), sc_in, mk.z));
                sr[c][e + 3] = __float_as_uint(fmaf(__uint_as_float(sr[c][e + 3]), sc_in, mk.w));
              }
          }
        }
        // keys of this tile that at least one row of this warp can see, in 32-key chunks: the others cost no exponentials
        int lim = it.len - k0;
        if (p.causal) lim = min(lim, it.q0 + quad * 32 + 32 - k0);
        const int live = tile_dead ? 0 : (min(lim, KT) + 31) >> 5;
        if ((k0 + KT > it.len) || (p.causal && k0 + KT - 1 > it.q0 + quad * 32)) {  // edge tile: keys past the end / above the diagonal
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int key = k0 + c * 32 + e;
              if (key >= it.len || (p.causal && key > qrow)) sr[c][e] = 0xff800000u;  // -inf
            }
        }
        // Reference maximum: taken on the first tile; later tiles keep it unless the guard below trips.
        bool need_max = (j == 0);
        float rs0, rs1;
        uint32_t pk[2][32];
        while (true) {
          if (need_max) {
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < 32; ++e)
#pragma unroll
              for (int c = 0; c < 4; ++c) mx[c] = fmaxf(mx[c], __uint_as_float(sr[c][e]));
            const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sc);
            if (j > 0) {
              // O holds tiles < j once PV(g-1) has completed; nothing writes it again until this warp releases P_g
              if (!__all_sync(0xffffffffu, mbar_wait(o_done(s), (g - 1) & 1u, abort_flag))) { ok = false; break; }
              tc_fence_after();
              const float corr = ex2(m_used - m_new);  // 2^-inf = 0 covers a row that had seen no live key yet
              l_run *= corr;
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                tmem_ld32_issue(to + (uint32_t)(c * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * corr);
                tmem_st32(to + (uint32_t)(c * 32), r);
              }
            }
            m_used = m_new;
          }
          const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
          rs0 = 0.f;
          rs1 = 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t* dst = &pk[c >> 1][(c & 1) * 16];
            if (c < live) {  // warp-uniform
#pragma unroll
              for (int e = 0; e < 32; e += 4) {
                const float a0 = ex2(fmaf(__uint_as_float(sr[c][e]), sc, -m_sub)), a1 = ex2(fmaf(__uint_as_float(sr[c][e + 1]), sc, -m_sub));
                const float a2 = ex2(fmaf(__uint_as_float(sr[c][e + 2]), sc, -m_sub)), a3 = ex2(fmaf(__uint_as_float(sr[c][e + 3]), sc, -m_sub));
                rs0 += a0 + a1;
                rs1 += a2 + a3;
                dst[e >> 1] = pack2<T>(a0, a1);
                dst[(e >> 1) + 1] = pack2<T>(a2, a3);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e) dst[e] = 0u;
            }
          }
          // every probability is below the row sum: under the limit none of them leaves the 16-bit range
          if (need_max || !__any_sync(0xffffffffu, !(rs0 + rs1 < kRowSumLimit))) break;
          need_max = true;  // a score far above the reference: redo this tile against its true maximum
        }
        if (!ok) break;
        l_run += rs0 + rs1;
        // P is read by PV(g-1), which is issued after the scores of this tile: it must have completed before P_g lands
        if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(o_done(s), (g - 1) & 1u, abort_flag))) { ok = false; break; }
        tmem_st32(tp, pk[0]);
        tmem_st32(tp + 32u, pk[1]);
        tmem_st_wait();
        tc_fence_before();  // O rescaled, P_g written
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready(s));
      }
      if (!ok) break;
      pend = true;
      pend_inv = 1.0f / l_run;
      pend_rows = it.len - it.q0 - quad * 32;
      pend_qb = (int)(nq & 1u);
      pend_base = static_cast<T*>(p.out) + (long long)(it.tok0 + it.q0 + quad * 32) * H + it.head * D;
    }
    if (ok && pend) flush_output();  // the stream's last item
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, (int)TTB_ERR_DEVICE_WAIT);
  if (threadIdx.x == 0) {  // the last CTA to finish leaves the work counters at zero for the next launch
    __threadfence();
    if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
    }
  }
}

}  // namespace

namespace ttb {

// TTB_ATTN_TC: 0 = never use the tensor-memory kernel, 2 = use it whenever it can run, anything else / unset = let the
// dispatcher choose by shape. Read on every call.
int attention_tc_mode() {
  const char* e = getenv("TTB_ATTN_TC");
  if (e && e[0] == '0') return 0;
  if (e && e[0] == '2') return 2;
  return 1;
}

// Launches the tcgen05 attention kernel. qkv is [tokens, 3*heads*64] in fp16/bf16; mask is null or an additive fp32 mask
// with one row of keys per sequence (masks with a row per query use the mma.sync kernel). Returns TTB_ERR_UNSUPPORTED when
// the batch does not fit the schedule tables or the tensor map cannot be encoded, so the caller can fall back.
int attention_tc_launch(ttb_ctx* ctx, int dtype, const void* qkv, int64_t tokens, const int32_t* cu, int64_t B, int64_t max_seqlen,
                        int64_t heads, const float* mask, int64_t mask_batch_stride, int causal, float scale, void* out) {
  if (B > kMaxB || B < 1 || heads < 1) return TTB_ERR_UNSUPPORTED;
  const int64_t H = heads * D;
  CUtensorMap tm;
  if (!encode_tile_map(&tm, qkv, 2, dtype == TTB_BF16, (uint64_t)tokens, (uint64_t)(3 * H), (uint64_t)(3 * H), 128))
    return TTB_ERR_UNSUPPORTED;
  static const int staged = [] { const char* e = getenv("TTB_ATTN_STAGED"); return (e && e[0] == '0') ? 0 : 1; }();
  Params p{out, cu, (int)B, (int)heads, causal ? 1 : 0, scale, ctx->d_status, ctx->d_status + 1, staged, mask, (long long)mask_batch_stride};
  // upper bound of the item count from what the host knows; a CTA runs two streams, idle CTAs leave after the tables
  const int64_t tiles_bound = std::min<int64_t>(tokens / QT + B, B * ((max_seqlen + QT - 1) / QT));
  const int64_t items_bound = std::max<int64_t>(1, tiles_bound * heads);
  dim3 grid((unsigned)std::min<int64_t>(ctx->sm_count, (items_bound + 1) / 2));
  static bool configured[64] = {};
  const int dev = ctx->device < 64 ? ctx->device : 63;
  if (!configured[dev]) {
    TTB_CUDA(ctx, cudaFuncSetAttribute(attention_tc_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    TTB_CUDA(ctx, cudaFuncSetAttribute(attention_tc_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    TTB_CUDA(ctx, cudaFuncSetAttribute(attention_tc_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    TTB_CUDA(ctx, cudaFuncSetAttribute(attention_tc_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured[dev] = true;
  }
  if (mask) {
    if (dtype == TTB_F16) launch_pdl(attention_tc_kernel<__half, true>, grid, dim3(kThreads), SMEM_BYTES, ctx->stream, tm, p);
    else launch_pdl(attention_tc_kernel<__nv_bfloat16, true>, grid, dim3(kThreads), SMEM_BYTES, ctx->stream, tm, p);
  } else {
    if (dtype == TTB_F16) launch_pdl(attention_tc_kernel<__half, false>, grid, dim3(kThreads), SMEM_BYTES, ctx->stream, tm, p);
    else launch_pdl(attention_tc_kernel<__nv_bfloat16, false>, grid, dim3(kThreads), SMEM_BYTES, ctx->stream, tm, p);
  }
  return launched(ctx, mask ? "attention_tc_mask" : "attention_tc");
}

}  // namespace ttb
