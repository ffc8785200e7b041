// Forward attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head dim <= 256.
//
// Persistent kernel: one CTA per SM draws work items (batch, head, block of 256 query rows[, KV split])
// from a heaviest-first list, either through a global counter (dynamic, when the caller provides one)
// or round-robin.  An item is two 128-row query tiles that take turns on the tensor pipe (head dims
// above 128: one tile, because O alone fills 256 TMEM columns).
// Warp roles (384 threads):
//   warps 0-3    softmax of tile 0  (one thread per query row; tcgen05.ld 32x32b gives a thread its row), and at
//                the end of an item its epilogue: O leaves tensor memory in one round trip (which frees it for
//                the next item's first PV, already queued behind this item's last one), then O / l and LSE go to
//                global memory while the first S of the next item is being computed
//   warps 4-7    the same for tile 1
//   warp  8      TMA producer: Q tiles per item, then K(j), V(j), K(j+1), ... through a ring of slots
//                that runs on across items
//   warp  9      MMA issuer: the warp stays converged, one elected lane issues every tcgen05.mma
//   warp  10     scheduler: fetches item numbers ahead of use into a small ring
//   warp  11     owns the TMEM allocation
// TMEM columns (fp32): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).  P (16-bit) is
// written over the first 64 columns of its S and fed to the PV MMA as the TMEM A operand.
// MMA order  S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) | ...  so that while one tile is in its
// softmax the other tile's two MMAs keep the tensor pipe busy; the first S of the next item follows
// the last PV of the current one in the same stream.  P is handed over in two halves of 64 keys,
// each followed by its four k-steps of PV.
// Softmax works in the exp2 domain with a lazily updated reference maximum: O and the row sum are
// only rescaled when the running maximum has grown by more than 2^8, which keeps the (expensive)
// TMEM round trip of O off the common path; the final O/l and LSE do not depend on that choice.
// Masks are applied per 32-column chunk: a chunk that a whole warp sees entirely is left alone, one
// that no row of the warp sees is skipped (no exponentials), only the chunks on the mask boundary
// are tested element by element.
//
// Split-KV (num_splits > 1): an item also names a range of key blocks; its normalised partial O and
// its LSE go to the fp32 workspaces and combine.cu merges them (flash_api.cpp:373-389,
// flash_fwd_launch_template.h:70-138).
//
// Same math as compute_attn_1rowblock (csrc/flash_attn/src/flash_fwd_kernel.h:74-580); mask rule of
// csrc/flash_attn/src/softmax.h:142-179; O = 0 and LSE = +inf for rows without a visible key.
#include <cstdlib>
#include <type_traits>

#include "../fa_common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace fa {

using namespace ptx;

StatusRef status_ref(bool may_allocate);

namespace {

constexpr int kBM = 128;  // rows per query tile
constexpr int kBN = 128;  // keys per K/V tile
constexpr int kChunkBytes = 128 * 128;  // [128 rows][64 x 16-bit]: one swizzled TMA box
constexpr float kRescaleThreshold = 8.f;
constexpr int kThreads = 384;
constexpr int kWarpTma = 8, kWarpMma = 9, kWarpSched = 10, kWarpTmem = 11;
constexpr int kSchedSlots = 4;
#ifndef FA_FWD_REGS_SOFTMAX
#define FA_FWD_REGS_SOFTMAX 208
#define FA_FWD_REGS_OTHER 88
#endif
// Registers per thread by role (setmaxnreg).  A softmax thread keeps its whole row of S (128 values) in registers.
// The CTA starts with 168 registers per thread (65536 / 384, rounded down to a multiple of 8) and can only
// redistribute THAT pool: an increase that the other warps' decreases do not cover would wait forever.
constexpr int kRegsSoftmax = FA_FWD_REGS_SOFTMAX, kRegsOther = FA_FWD_REGS_OTHER;
constexpr int kRegsAtLaunch = (65536 / kThreads) / 8 * 8;
static_assert(256 * kRegsSoftmax + 128 * kRegsOther <= kThreads * kRegsAtLaunch, "register pool of the CTA");
static_assert(kRegsOther <= kRegsAtLaunch && kRegsSoftmax >= kRegsAtLaunch, "setmaxnreg directions");

enum WaitCode { W_QFULL = 11, W_KVFULL = 12, W_KVEMPTY = 13, W_SFULL = 14, W_PFULL = 15, W_OFULL = 16,
                W_QEMPTY = 17, W_OFINAL = 18, W_OEMPTY = 19, W_STATS = 10, W_SCHED = 9 };

template <int DH>
struct Cfg {
  static constexpr int NCHUNK = DH / 64;
  static constexpr int TILE_BYTES = NCHUNK * kChunkBytes;
  // Head dims up to 128: two 128-row query tiles per item ping-pong on the tensor pipe.  Up to 256: O alone
  // needs 256 TMEM columns and a tile is 64 KiB, so one query tile per item and a 2-slot (K, V) ring.
  static constexpr int NT = DH > 128 ? 1 : 2;
  static constexpr int STAGES = DH > 128 ? 2 : (DH == 128 ? 4 : 8);
  static constexpr int SMEM_TILES = (NT + STAGES) * TILE_BYTES;
  // barriers: q full/empty [2+2], kv full/empty [2*STAGES], s full [2], p full [2][2], o full [2], o final [2],
  // o empty [2], sched full/empty [2*kSchedSlots]
  static constexpr int NBAR = 4 + 2 * STAGES + 2 + 4 + 2 + 2 + 2 + 2 * kSchedSlots;
  static constexpr int OFF_BAR = SMEM_TILES;
  static constexpr int OFF_SCHED = OFF_BAR + NBAR * 8;           // kSchedSlots ints
  static constexpr int OFF_ABORT = OFF_SCHED + kSchedSlots * 4;  // tmem ptr / abort block
  static constexpr int SMEM_BYTES = OFF_ABORT + 32 + 1024;       // + align slack
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S0 = 0, COL_S1 = 128, COL_O0 = 256, COL_O1 = 256 + DH;
  static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA");
};

struct FwdTcParams {
  CUtensorMap tq, tk, tv;
  FaFwdArgs a;
  StatusRef status;
  // work list: item -> (split, section of `sec_pairs` (batch, head) pairs, row block heaviest first, pair)
  int32_t n_items, n_m, n_pairs, sec_pairs, num_splits, blocks_per_split;
};

template <typename T>
struct Fmt;
template <>
struct Fmt<__half> {
  static constexpr int kIdesc = 0;
};
template <>
struct Fmt<__nv_bfloat16> {
  static constexpr int kIdesc = 1;
};

// One work item as every role sees it.
struct Item {
  SeqInfo si;
  int b, h, hk, split, m_base;
  int lo[2], hi[2];  // key blocks [lo, hi) of each tile (already cut to the item's split)
  int J_lo, J_hi;    // their union
  bool live;         // false: the row block lies past the end of this sequence, every role skips it
  bool active[2];    // tile has rows of the sequence
};

template <int NT>
__device__ __forceinline__ Item decode_item(const FwdTcParams& P, int idx) {
  const FaFwdArgs& a = P.a;
  Item it;
  int r = idx;
  it.split = 0;
  if (P.num_splits > 1) {
    it.split = idx % P.num_splits;
    r = idx / P.num_splits;
  }
  const int sec_items = P.sec_pairs * P.n_m;
  const int sec = r / sec_items, w = r - sec * sec_items;
  const int pairs_here = min(P.sec_pairs, P.n_pairs - sec * P.sec_pairs);
  const int mrank = w / pairs_here, pr = sec * P.sec_pairs + (w - mrank * pairs_here);
  const int mblk = P.n_m - 1 - mrank;  // heaviest row blocks (bottom rows of a causal mask) first
  it.b = pr / a.heads;
  it.h = pr - it.b * a.heads;
  it.hk = it.h / (a.heads / a.heads_k);
  it.si = seq_info(a.cu_seqlens_q, a.cu_seqlens_k, nullptr, nullptr, a.seqlen_q, a.seqlen_k, a.use_mask_shift,
                   a.mask_shift, it.b);
  it.m_base = mblk * NT * kBM;
  it.live = it.m_base < it.si.sq;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int m0 = it.m_base + t * kBM;
    it.active[t] = t < NT && m0 < it.si.sq;
    it.lo[t] = it.hi[t] = 0;
    if (it.active[t]) {
      key_block_range(m0, kBM, kBN, it.si.sk, it.si.shift, a.window_left, a.window_right, it.lo[t], it.hi[t]);
      if (P.num_splits > 1) {
        const int s_lo = it.split * P.blocks_per_split, s_hi = s_lo + P.blocks_per_split;
        it.lo[t] = max(it.lo[t], s_lo);
        it.hi[t] = min(it.hi[t], s_hi);
        if (it.hi[t] <= it.lo[t]) it.lo[t] = it.hi[t] = 0;
      }
    }
  }
  const bool h0 = it.hi[0] > it.lo[0], h1 = it.hi[1] > it.lo[1];
  if (h0 && h1) {
    it.J_lo = min(it.lo[0], it.lo[1]);
    it.J_hi = max(it.hi[0], it.hi[1]);
  } else if (h0) {
    it.J_lo = it.lo[0];
    it.J_hi = it.hi[0];
  } else {
    it.J_lo = it.lo[1];
    it.J_hi = it.hi[1];
  }
  return it;
}

template <typename T, int DH>
__global__ void __launch_bounds__(kThreads, 1) fwd_tc_kernel(const __grid_constant__ FwdTcParams P) {
  using C = Cfg<DH>;
  constexpr int NT = C::NT;
  const FaFwdArgs& a = P.a;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_addr(smem);
  const uint32_t sQ = s_base;                          // NT tiles
  const uint32_t sKV = s_base + NT * C::TILE_BYTES;     // STAGES slots
  const uint32_t bar0 = s_base + C::OFF_BAR;
  constexpr int S = C::STAGES;
  const uint32_t b_qfull = bar0, b_qempty = bar0 + 8 * 2, b_kvfull = bar0 + 8 * 4, b_kvempty = bar0 + 8 * (4 + S),
                 b_sfull = bar0 + 8 * (4 + 2 * S), b_pfull = bar0 + 8 * (6 + 2 * S), b_ofull = bar0 + 8 * (10 + 2 * S),
                 b_ofinal = bar0 + 8 * (12 + 2 * S), b_oempty = bar0 + 8 * (14 + 2 * S), b_scfull = bar0 + 8 * (16 + 2 * S),
                 b_scempty = bar0 + 8 * (16 + 2 * S + kSchedSlots);
  static_assert(16 + 2 * S + 2 * kSchedSlots == C::NBAR, "barrier count");
  volatile int* sched_item = reinterpret_cast<volatile int*>(smem + C::OFF_SCHED);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_ABORT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_ABORT + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kConsumers = NT * 4 + 2;  // softmax, TMA and MMA warps read the item ring

  if (threadIdx.x == 0) {
    abort_init(abort_flag, P.status);
    for (int t = 0; t < 2; ++t) {
      mbar_init(b_qfull + 8 * t, 1);
      mbar_init(b_qempty + 8 * t, 1);
      mbar_init(b_sfull + 8 * t, 1);
      mbar_init(b_pfull + 8 * (2 * t), 4);
      mbar_init(b_pfull + 8 * (2 * t + 1), 4);
      mbar_init(b_ofull + 8 * t, 1);
      mbar_init(b_ofinal + 8 * t, 1);
      mbar_init(b_oempty + 8 * t, 4);
    }
    for (int s = 0; s < S; ++s) {
      mbar_init(b_kvfull + 8 * s, 1);
      mbar_init(b_kvempty + 8 * s, 1);
    }
    for (int s = 0; s < kSchedSlots; ++s) {
      mbar_init(b_scfull + 8 * s, 1);
      mbar_init(b_scempty + 8 * s, kConsumers);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == kWarpTmem) {
    tmem_alloc(smem_addr(const_cast<uint32_t*>(tmem_ptr_smem)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;

  const float scale_log2 = a.softmax_scale * kLog2e;
  const int64_t rows_total = (int64_t)a.batch * a.heads * a.seqlen_q;  // row pitch of the split workspaces

  // Item number k of this CTA, as published by the scheduler warp (-1: no more work).  Called by whole warps.
  auto next_item = [&](int k, bool& ok) -> int {
    const int slot = k % kSchedSlots;
    ok = mbar_wait(b_scfull + 8 * slot, (k / kSchedSlots) & 1, W_SCHED, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    const int item = ok ? sched_item[slot] : -1;
    __syncwarp();
    if (lane == 0) mbar_arrive(b_scempty + 8 * slot);
    return item;
  };

  if (warp < 4 * NT) {
    // ------------------------------------------------------------------ softmax warpgroups
    setmaxnreg_inc<kRegsSoftmax>();
    const int t = warp >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_off + (t ? C::COL_S1 : C::COL_S0);
    const uint32_t tO = tmem + lane_off + (t ? C::COL_O1 : C::COL_O0);
    const uint64_t scale2 = pack2(scale_log2, scale_log2);
    uint32_t n_s = 0;   // S blocks of this tile consumed so far (phase of s_full / p_full / o_full)
    uint32_t n_of = 0;  // items whose O of this tile was taken out of tensor memory
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int idx = next_item(k, ok);
      if (idx < 0) break;
      const Item it = decode_item<NT>(P, idx);
      if (!it.live) continue;
      const SeqInfo& si = it.si;
      const int m0 = it.m_base + t * kBM;
      const int row = m0 + row_in_tile;
      float m_used = -INFINITY;
      uint64_t l_sum2 = pack2(0.f, 0.f);  // two running partial row sums (even / odd columns)
      // first / last visible key of this row (inclusive)
      int col_first = 0, col_last = si.sk - 1;
      if (a.window_right >= 0) col_last = min(col_last, row + si.shift + a.window_right);
      if (a.window_left >= 0) col_first = max(col_first, row + si.shift - a.window_left);

      for (int j = it.lo[t]; j < it.hi[t] && ok; ++j) {
        const bool first_block = j == it.lo[t];
        ok = mbar_wait(b_sfull + 8 * t, n_s & 1, W_SFULL, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const int n0 = j * kBN;
        const bool need_mask = (n0 + kBN - 1 >= si.sk) ||
                               (a.window_right >= 0 && n0 + kBN - 1 > m0 + si.shift + a.window_right) ||
                               (a.window_left >= 0 && n0 < m0 + kBM - 1 + si.shift - a.window_left);
        // One block of the online softmax.  MASKED = false is the straight-line version for blocks that every row
        // sees entirely; MASKED = true classifies each 32-column chunk for the warp: bit q of `none` = no row of
        // this warp sees chunk q (no maximum, no exponentials, P = 0), bit q of `part` = the mask boundary crosses
        // it (tested element by element), otherwise the chunk is fully visible.
        auto block = [&](auto masked_tag) -> bool {
          constexpr bool MASKED = decltype(masked_tag)::value;
          uint32_t none = 0, part = 0;
          const int c_lo = col_first - n0, c_hi = col_last - n0;
          if (MASKED) {
            // the bounds do not decrease with the row index: lane 0 / lane 31 hold the extremes of the warp
            const int lo_min = __shfl_sync(0xffffffffu, c_lo, 0), lo_max = __shfl_sync(0xffffffffu, c_lo, 31);
            const int hi_min = __shfl_sync(0xffffffffu, c_hi, 0), hi_max = __shfl_sync(0xffffffffu, c_hi, 31);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int c0 = 32 * q;
              if (c0 > hi_max || c0 + 31 < lo_min)
                none |= 1u << q;
              else if (!(c0 >= lo_max && c0 + 31 <= hi_min))
                part |= 1u << q;
            }
          }
          // the whole row of S in registers: one round trip to tensor memory
          uint32_t su[4][32];
          tmem_ld32(tS + 0, su[0]);
          tmem_ld32(tS + 32, su[1]);
          tmem_ld32(tS + 64, su[2]);
          tmem_ld32(tS + 96, su[3]);
          tmem_wait_ld();
          if (MASKED) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (part & (1u << q)) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (!(32 * q + i >= c_lo && 32 * q + i <= c_hi)) su[q][i] = 0xff800000u;  // -inf
              }
            }
          }
          // row maximum: four chains of three-input max
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (!MASKED || !(none & (1u << q))) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                mx0 = max3(mx0, __uint_as_float(su[q][i]), __uint_as_float(su[q][i + 1]));
                mx1 = max3(mx1, __uint_as_float(su[q][i + 2]), __uint_as_float(su[q][i + 3]));
                mx2 = max3(mx2, __uint_as_float(su[q][i + 4]), __uint_as_float(su[q][i + 5]));
                mx3 = max3(mx3, __uint_as_float(su[q][i + 6]), __uint_as_float(su[q][i + 7]));
              }
            }
          }
          const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
          const float m_cand = fmaxf(m_used, m_blk);
          const bool grow = m_cand > m_used + kRescaleThreshold;  // also true when m_used is -inf and m_cand is finite
          if (!first_block && __any_sync(0xffffffffu, grow)) {
            // O and l are relative to m_used: move them to the new reference (PV of the block before must be done)
            if (!mbar_wait(b_ofull + 8 * t, (n_s - 1) & 1, W_OFULL, abort_flag)) return false;
            tc_fence_after();
            const float f = grow ? fast_exp2(m_used - m_cand) : 1.f;
#pragma unroll
            for (int c0 = 0; c0 < DH; c0 += 16) {
              uint32_t o[16];
              tmem_ld16(tO + c0, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
              tmem_st16(tO + c0, o);
            }
            l_sum2 = fma2(l_sum2, pack2(f, f), pack2(0.f, 0.f));
          }
          if (grow) m_used = m_cand;
          const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
          const uint64_t neg_m2 = pack2(neg_m, neg_m);
          // P = exp2(S * scale - m), 16-bit, over the first 64 columns of S, handed to the MMA warp in two halves
          // of 64 keys, so that the first four k-steps of PV run while the second half is still being computed
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t pu[32];
#pragma unroll
            for (int qq = 0; qq < 2; ++qq) {
              const int q = half * 2 + qq;
              if (MASKED && (none & (1u << q))) {
#pragma unroll
                for (int i = 0; i < 16; ++i) pu[qq * 16 + i] = 0u;
              } else {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  const uint64_t x = fma2(pack2u(su[q][i], su[q][i + 1]), scale2, neg_m2);
                  float x0, x1;
                  unpack2(x, x0, x1);
                  const float e0 = ex2(x0), e1 = ex2(x1);
                  l_sum2 = add2(l_sum2, pack2(e0, e1));
                  pu[qq * 16 + (i >> 1)] = Pack<T>::two(e0, e1);
                }
              }
            }
            tmem_st32(tS + half * 32, pu);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_pfull + 8 * (2 * t + half));
          }
          return true;
        };
        ok = need_mask ? block(std::true_type{}) : block(std::false_type{});
        if (!ok) break;
        ++n_s;
      }
      if (!ok) break;
      // ---- epilogue of the item for this tile: LSE, then O / l
      float la, lb;
      unpack2(l_sum2, la, lb);
      const float l_sum = la + lb;
      const bool empty = !(l_sum > 0.f) || m_used == -INFINITY;
      const float inv = empty ? 0.f : 1.f / l_sum;
      const float lse = empty ? INFINITY : (m_used + log2f(l_sum)) * kLn2;
      const bool store = it.active[t] && row < si.sq;
      const int nblk_t = it.hi[t] - it.lo[t];
      const int64_t ridx = ((int64_t)it.b * a.heads + it.h) * a.seqlen_q + row;  // split workspaces are not packed
      if (store) {
        if (P.num_splits > 1)
          a.lse_accum[(int64_t)it.split * rows_total + ridx] = empty ? -INFINITY : lse;
        else
          a.softmax_lse[((int64_t)it.b * a.heads + it.h) * a.lse_seqlen + row] = lse;
      }
      if (!it.active[t]) continue;  // warp-uniform (a tile is 128 rows): no rows of the sequence in this tile
      if (nblk_t > 0) {
        ok = mbar_wait(b_ofinal + 8 * t, n_of & 1, W_OFINAL, abort_flag);
        if (!ok) break;
        ++n_of;
        tc_fence_after();
      }
      float* oa = P.num_splits > 1 ? a.out_accum + ((int64_t)it.split * rows_total + ridx) * a.head_dim : nullptr;
      T* og = reinterpret_cast<T*>(a.out.ptr) + si.q_batch * a.out.stride_b + (si.q_row0 + row) * a.out.stride_s +
              (int64_t)it.h * a.out.stride_h;
      constexpr int OB = DH < 128 ? DH : 128;  // columns of O taken out of tensor memory per round trip
#pragma unroll
      for (int c0 = 0; c0 < DH; c0 += OB) {
        uint32_t o[OB];
        if (nblk_t > 0) {
#pragma unroll
          for (int c = 0; c < OB; c += 32) tmem_ld32(tO + c0 + c, *reinterpret_cast<uint32_t(*)[32]>(&o[c]));
          tmem_wait_ld();
          if (c0 + OB == DH) {
            // O is in registers: the next item's first PV (queued behind this item's last one) may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_oempty + 8 * t);
          }
        } else {
#pragma unroll
          for (int i = 0; i < OB; ++i) o[i] = 0u;
        }
        if (!store) continue;
        if (P.num_splits > 1) {
#pragma unroll
          for (int i = 0; i < OB; i += 4)
            if (c0 + i < a.head_dim)
              *reinterpret_cast<float4*>(oa + c0 + i) =
                  make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv, __uint_as_float(o[i + 2]) * inv,
                              __uint_as_float(o[i + 3]) * inv);
        } else {
#pragma unroll
          for (int i = 0; i < OB; i += 8) {
            if (c0 + i < a.head_dim) {
              uint4 pk;
              pk.x = Pack<T>::two(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
              pk.y = Pack<T>::two(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              pk.z = Pack<T>::two(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              pk.w = Pack<T>::two(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(og + c0 + i) = pk;
            }
          }
        }
      }
    }
  } else if (warp >= 4 * NT && warp < 8) {
    setmaxnreg_dec<kRegsOther>();  // head dims above 128: the second softmax warpgroup has no tile
  } else {
    setmaxnreg_dec<kRegsOther>();
    if (warp == kWarpSched) {
      // ---------------------------------------------------------------- scheduler
      // Item numbers are fetched ahead of use.  The first item of a CTA is its block index; the others come from
      // the caller's counter (dynamic) or follow round-robin.  The CTA that fetches last resets the counter pair.
      if (lane == 0) {
        bool ok = true;
        for (int k = 0; ok; ++k) {
          const int slot = k % kSchedSlots;
          if (k >= kSchedSlots) {
            ok = mbar_wait(b_scempty + 8 * slot, ((k / kSchedSlots) - 1) & 1, W_SCHED, abort_flag, 3);
            if (!ok) break;
          }
          int item;
          if (k == 0) {
            item = blockIdx.x;
          } else if (a.tile_counter != nullptr) {
            item = atomicAdd(a.tile_counter, 1) + (int)gridDim.x;
          } else {
            item = blockIdx.x + k * (int)gridDim.x;
          }
          if (item >= P.n_items) item = -1;
          sched_item[slot] = item;
          mbar_arrive(b_scfull + 8 * slot);
          if (item < 0) break;
        }
        if (a.tile_counter != nullptr) {
          __threadfence();
          if (atomicAdd(a.tile_counter + 1, 1) == (int)gridDim.x - 1) {
            a.tile_counter[0] = 0;
            a.tile_counter[1] = 0;
            __threadfence();
          }
        }
      }
    } else if (warp == kWarpTma) {
      // ---------------------------------------------------------------- TMA producer
      uint32_t kv_idx = 0;           // K / V tiles loaded so far (ring position)
      uint32_t n_q[2] = {0, 0};      // items whose Q tile t was loaded
      bool ok = true;
      if (lane == 0) {
        prefetch_tensormap(&P.tq);
        prefetch_tensormap(&P.tk);
        prefetch_tensormap(&P.tv);
      }
      for (int k = 0; ok; ++k) {
        const int idx = next_item(k, ok);
        if (idx < 0) break;
        const Item it = decode_item<NT>(P, idx);
        const int nblk = it.J_hi - it.J_lo;
        if (!it.live || nblk <= 0) continue;
        if (lane == 0) {
          const int qrow = (int)it.si.q_row0 + it.m_base;
          const int qb = (int)it.si.q_batch, kb = (int)it.si.k_batch;
          for (int t = 0; t < NT && ok; ++t) {
            if (it.hi[t] <= it.lo[t]) continue;
            if (n_q[t] > 0) ok = mbar_wait(b_qempty + 8 * t, (n_q[t] - 1) & 1, W_QEMPTY, abort_flag, 2);
            if (!ok) break;
            ++n_q[t];
            mbar_expect_tx(b_qfull + 8 * t, C::TILE_BYTES);
            for (int c = 0; c < C::NCHUNK; ++c)
              tma_load_4d(sQ + t * C::TILE_BYTES + c * kChunkBytes, &P.tq, b_qfull + 8 * t, c * 64, qrow + t * kBM, it.h, qb);
          }
          for (int i = 0; i < 2 * nblk && ok; ++i, ++kv_idx) {
            const uint32_t slot = kv_idx % S, round = kv_idx / S;
            ok = mbar_wait(b_kvempty + 8 * slot, (round & 1) ^ 1, W_KVEMPTY, abort_flag, 2);
            if (!ok) break;
            const int j = it.J_lo + (i >> 1);
            const CUtensorMap* tm = (i & 1) ? &P.tv : &P.tk;
            mbar_expect_tx(b_kvfull + 8 * slot, C::TILE_BYTES);
            for (int c = 0; c < C::NCHUNK; ++c)
              tma_load_4d(sKV + slot * C::TILE_BYTES + c * kChunkBytes, tm, b_kvfull + 8 * slot, c * 64,
                          (int)it.si.k_row0 + j * kBN, it.hk, kb);
          }
        }
        // n_q / kv_idx live in lane 0 only; the other lanes just follow the item sequence
        ok = __all_sync(0xffffffffu, ok);
      }
    } else if (warp == kWarpMma) {
      // ---------------------------------------------------------------- MMA issuer
      // The whole warp runs the loop (see mma_ss_w); one elected lane issues.
      constexpr uint32_t idesc_s = make_idesc(kBM, kBN, Fmt<T>::kIdesc, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(kBM, DH, Fmt<T>::kIdesc, 0, 1);
      bool ok = true;
      // One descriptor is built (Q tile 0, K-major); every other operand differs from it only in the
      // low word: the address field (+ byte offset >> 4) and, for MN-major reads, the LBO field.
      const uint64_t d_base = smem_desc_sw128(sQ, 16, 1024);
      const uint32_t d_lo = (uint32_t)d_base, d_hi = (uint32_t)(d_base >> 32);
      auto dsc = [&](uint32_t lo_add) { return ((uint64_t)d_hi << 32) | (uint64_t)(d_lo + lo_add); };
      constexpr uint32_t kMn = (uint32_t)((kChunkBytes - 16) >> 4) << 16;  // K-major -> MN-major (LBO = chunk stride)
      constexpr uint32_t kTile16 = C::TILE_BYTES >> 4, oKV = (NT * C::TILE_BYTES) >> 4;
      uint32_t kv_idx = 0;          // K / V tiles consumed so far (ring position)
      uint32_t n_q[2] = {0, 0};     // items whose Q tile t was consumed
      uint32_t n_p[2] = {0, 0};     // P blocks of tile t consumed (phase of p_full)
      uint32_t n_o[2] = {0, 0};     // items whose O of tile t was completed (phase of o_empty)
      auto slot_of = [&](uint32_t i) { return i % S; };
      auto par_of = [&](uint32_t i) { return (uint32_t)((i / S) & 1); };
      struct Rng {  // what the issuer needs of an item: key blocks [lo, hi) per tile and their union
        int lo[2], hi[2], J_lo, J_hi;
      };
      auto in_range = [&](const Rng& it, int t, int j) { return j >= it.lo[t] && j < it.hi[t]; };
      // S_t = Q_t K^T from the K tile in `slot`; `last` = it is the tile's last block of the item: Q_t may be replaced
      auto issue_s = [&](int t, uint32_t slot, bool last) {
        const uint32_t d = tmem + (t ? C::COL_S1 : C::COL_S0);
        const uint32_t a_lo = t ? kTile16 : 0u, b_lo = oKV + slot * kTile16;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t off = (uint32_t)(((kk >> 2) * kChunkBytes + (kk & 3) * 32) >> 4);
          mma_ss_w(d, dsc(a_lo + off), dsc(b_lo + off), idesc_s, kk > 0);
        }
        tc_commit_w(b_sfull + 8 * t);
        if (last) tc_commit_w(b_qempty + 8 * t);
      };
      // PV in two halves of four k-steps: the softmax warps hand over P in two pieces (keys 0-63, then 64-127)
      auto issue_pv_half = [&](int t, uint32_t slot, bool first, int half) {
        const uint32_t d = tmem + (t ? C::COL_O1 : C::COL_O0);
        const uint32_t pa = tmem + (t ? C::COL_S1 : C::COL_S0);
        const uint32_t b_lo = oKV + slot * kTile16 + kMn;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int kk = half * 4 + k4;
          mma_ts_w(d, pa + kk * 8, dsc(b_lo + (uint32_t)((kk * 2048) >> 4)), idesc_o, (!first) || kk > 0);
        }
      };
      // First S of an item: Q tiles and K(J_lo) must have landed.  Consumes one ring tile.
      auto start_item = [&](const Rng& it) {
        for (int t = 0; t < NT && ok; ++t) {
          if (it.hi[t] <= it.lo[t]) continue;
          ok = mbar_wait_w(b_qfull + 8 * t, n_q[t] & 1, W_QFULL, abort_flag);
          ++n_q[t];
        }
        if (ok) ok = mbar_wait_w(b_kvfull + 8 * slot_of(kv_idx), par_of(kv_idx), W_KVFULL, abort_flag);
        if (!ok) return;
        tc_fence_after();
        for (int t = 0; t < NT; ++t)
          if (in_range(it, t, it.J_lo)) issue_s(t, slot_of(kv_idx), it.J_lo == it.hi[t] - 1);
        tc_commit_w(b_kvempty + 8 * slot_of(kv_idx));
        ++kv_idx;
      };
      // next item of this CTA that has key blocks (others are skipped by TMA and MMA alike)
      int k_sched = 0;
      Rng cur, nxt;
      auto fetch = [&](Rng& dst) -> bool {
        while (ok) {
          const int idx = next_item(k_sched++, ok);
          if (idx < 0) return false;
          const Item it = decode_item<NT>(P, idx);
          if (it.live && it.J_hi > it.J_lo) {
            dst.lo[0] = it.lo[0], dst.hi[0] = it.hi[0], dst.lo[1] = it.lo[1], dst.hi[1] = it.hi[1];
            dst.J_lo = it.J_lo, dst.J_hi = it.J_hi;
            return true;
          }
        }
        return false;
      };
      // A wait costs this warp 150+ cycles even when the barrier has long completed (a round trip to shared memory
      // between instructions that compete for issue slots with the softmax warps).  So each barrier is tested one
      // MMA group ahead of its use: the answer travels while the group before is being issued (the issue blocks at
      // the pace of the tensor pipe), and only a miss falls back to a real wait.  A hit stays valid until this warp
      // consumes the phase, because no producer can run more than one phase ahead of it.
      auto waitp = [&](uint32_t& hit, uint32_t bar, uint32_t par, int code) -> bool {
        const uint32_t h = hit;
        hit = 0;
        if (h) return true;
        return mbar_wait_w(bar, par, code, abort_flag);
      };
      uint32_t h_v = 0, h_k = 0, h_pa[2] = {0, 0}, h_pb[2] = {0, 0};
      bool have = fetch(cur);
      if (have) start_item(cur);
      while (have && ok) {
        const bool have_next = fetch(nxt);
        for (int j = cur.J_lo; j < cur.J_hi && ok; ++j) {
          const bool more = j + 1 < cur.J_hi;
          const uint32_t iv = kv_idx++;          // ring position of V(j)
          ok = waitp(h_v, b_kvfull + 8 * slot_of(iv), par_of(iv), W_KVFULL);
          uint32_t ik = 0;
          if (ok && more) {
            ik = kv_idx++;                       // ring position of K(j+1)
            ok = waitp(h_k, b_kvfull + 8 * slot_of(ik), par_of(ik), W_KVFULL);
          }
          h_k = 0;
          if (!ok) break;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            if (!ok) break;
            if (in_range(cur, t, j)) {
              const bool first = j == cur.lo[t];
              if (first && n_o[t] > 0) {  // the epilogue must have drained the O of the item before
                ok = mbar_wait_w(b_oempty + 8 * t, (n_o[t] - 1) & 1, W_OEMPTY, abort_flag);
                if (!ok) break;
              }
              ok = waitp(h_pa[t], b_pfull + 8 * (2 * t), n_p[t] & 1, W_PFULL);
              if (!ok) break;
              if (!h_pb[t]) h_pb[t] = mbar_test(b_pfull + 8 * (2 * t + 1), n_p[t] & 1);
              tc_fence_after();
              issue_pv_half(t, slot_of(iv), first, 0);
              ok = waitp(h_pb[t], b_pfull + 8 * (2 * t + 1), n_p[t] & 1, W_PFULL);
              if (!ok) break;
              if (NT == 2 && t == 0 && in_range(cur, 1, j)) h_pa[1] = mbar_test(b_pfull + 8 * 2, n_p[1] & 1);
              tc_fence_after();
              issue_pv_half(t, slot_of(iv), first, 1);
              ++n_p[t];
              tc_commit_w(b_ofull + 8 * t);
              if (j == cur.hi[t] - 1) {
                tc_commit_w(b_ofinal + 8 * t);
                ++n_o[t];
              }
            }
            if (t == NT - 1) tc_commit_w(b_kvempty + 8 * slot_of(iv));
            // tests whose answers travel while the (long) S group below is being issued
            if (NT == 2 && t == 0 && in_range(cur, 1, j)) h_pb[1] = mbar_test(b_pfull + 8 * 3, n_p[1] & 1);
            if (t == NT - 1 && more) {
              h_v = mbar_test(b_kvfull + 8 * slot_of(kv_idx), par_of(kv_idx));
              if (j + 2 < cur.J_hi) h_k = mbar_test(b_kvfull + 8 * slot_of(kv_idx + 1), par_of(kv_idx + 1));
              if (in_range(cur, 0, j + 1)) h_pa[0] = mbar_test(b_pfull, n_p[0] & 1);
            }
            if (more && in_range(cur, t, j + 1)) issue_s(t, slot_of(ik), j + 1 == cur.hi[t] - 1);
            if (more && t == NT - 1) tc_commit_w(b_kvempty + 8 * slot_of(ik));
          }
          // the first S of the next item goes out behind the last PV of this one
          if (ok && !more && have_next) start_item(nxt);
        }
        have = have_next;
        cur = nxt;
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == kWarpTmem) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <typename T, int DH>
int launch_fwd_tc(const FaFwdArgs& a, cudaStream_t st) {
  using C = Cfg<DH>;
  FwdTcParams P;
  P.a = a;
  const bool varlen = a.cu_seqlens_q != nullptr;
  const int64_t q_rows = varlen ? a.total_q : a.seqlen_q, k_rows = varlen ? a.total_k : a.seqlen_k;
  const int64_t nb = varlen ? 1 : a.batch;
  if (make_tmap_4d(&P.tq, a.q, a.dtype, q_rows, a.heads, nb, a.head_dim, kBM)) return 1;
  if (make_tmap_4d(&P.tk, a.k, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kBN)) return 1;
  if (make_tmap_4d(&P.tv, a.v, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kBN)) return 1;
  P.status = status_ref(true);
  // work list
  const int rows_per_item = C::NT * kBM;
  P.n_m = (a.seqlen_q + rows_per_item - 1) / rows_per_item;
  P.n_pairs = a.batch * a.heads;
  P.num_splits = a.num_splits > 1 ? a.num_splits : 1;
  const int n_blocks = (a.seqlen_k + kBN - 1) / kBN;
  P.blocks_per_split = (n_blocks + P.num_splits - 1) / P.num_splits;
  // a section is a run of (batch, head) pairs whose K and V stay in the L2 while their row blocks are worked
  // on: about 32 MB of distinct K / V (query heads of one KV head share theirs)
  const int group = a.heads / a.heads_k;
  const int64_t kv_bytes = 2ll * a.seqlen_k * a.head_dim * 2;
  int64_t kv_heads_per_sec = (32ll << 20) / (kv_bytes > 0 ? kv_bytes : 1);
  if (kv_heads_per_sec < 1) kv_heads_per_sec = 1;
  int64_t sec = kv_heads_per_sec * group;
  if (sec > P.n_pairs) sec = P.n_pairs;
  P.sec_pairs = (int)sec;
  const int64_t n_items = (int64_t)P.n_pairs * P.n_m * P.num_splits;
  if (n_items >= (1ll << 31)) {
    fa_host::set_error("fwd_tc_kernel: too many work items");
    return 1;
  }
  P.n_items = (int)n_items;
  auto kern = fwd_tc_kernel<T, DH>;
  static fa_host::DeviceOnce once;
  if (int rc = fa_host::raise_smem_limit(once, reinterpret_cast<const void*>(kern), C::SMEM_BYTES, "fwd_tc_kernel")) return rc;
  const int sms = fa_host::sm_count();
  dim3 grid(P.n_items < sms ? P.n_items : sms);
  kern<<<grid, kThreads, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("fwd_tc_kernel");
}

}  // namespace

bool fwd_tc_eligible(const FaFwdArgs& a) {
  if (a.head_dim > 256 || a.p_dropout > 0.f || a.s_dmask) return false;
  if (a.num_splits > 1 && a.cu_seqlens_q) return false;
  if (a.seqused_k || a.kv_batch_idx) return false;
  if (a.seqlen_k <= 0) return false;
  if (!tma_compatible(a.q) || !tma_compatible(a.k) || !tma_compatible(a.v)) return false;
  if ((reinterpret_cast<uintptr_t>(a.out.ptr) & 15) || a.out.stride_s % 8 || a.out.stride_h % 8 || a.out.stride_b % 8)
    return false;
  if (a.cu_seqlens_q && (a.total_q <= 0 || a.total_k <= 0)) return false;
  return encode_tiled_fn() != nullptr;
}

int fwd_tc(const FaFwdArgs& a, cudaStream_t st) {
  const bool bf = a.dtype == FA_DTYPE_BF16;
  if (a.head_dim <= 64) return bf ? launch_fwd_tc<__nv_bfloat16, 64>(a, st) : launch_fwd_tc<__half, 64>(a, st);
  if (a.head_dim <= 128) return bf ? launch_fwd_tc<__nv_bfloat16, 128>(a, st) : launch_fwd_tc<__half, 128>(a, st);
  return bf ? launch_fwd_tc<__nv_bfloat16, 256>(a, st) : launch_fwd_tc<__half, 256>(a, st);
}

}  // namespace fa
