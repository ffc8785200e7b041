// Backward attention on tcgen05 tensor cores (head dim <= 128), part 2 of 2: dQ.
//
// A work item is 128 query rows of one (batch, query head): Q and dO stay in shared memory, dQ in
// tensor memory, and the item walks every 128-key block those rows can see (bwd_tc.cu holds part 1,
// dK / dV, and says why the pass is split).  Same math as the dQ half of compute_dq_dk_dv_1colblock
// (csrc/flash_attn/src/flash_bwd_kernel.h:425-1112):
//   S   = Q K^T           (lanes = queries, columns = keys)             SS MMA  -> TMEM tS
//   dP  = dO V^T                                                         SS MMA  -> TMEM tdP
//   P   = exp2(S*scale*log2e - LSE*log2e)             one thread per query row, stays in registers
//   dS  = P o (dP - D)                                                   -> TMEM (16-bit, buffer g & 1)
//   dQ += dS K            A = dS from TMEM, B = K tile (MN-major)        -> TMEM tdQ
// S and dP are consumed into registers as soon as they are complete, so the tensor pipe computes
// S(j+1) and dP(j+1) while the compute warps are still working on block j; dS has two buffers of
// its own, so dQ(j) never holds up either of them.
//
// The kernel is persistent: one CTA per SM draws items from a global counter over a list ordered head by
// head (so that concurrent CTAs share K / V tiles in L2), heavy query blocks first.  All rings and barrier phases
// run on across items, so while the compute warps write out the dQ of one item the producer is
// already loading the next item's Q, dO and first K / V tiles and the tensor pipe computes its first
// S and dP: the launch, load latency, pipeline fill and drain that a CTA per item paid (several
// microseconds, a fifth of the time of a 2048-token causal problem) overlap with useful work.
//
// Warps: 0-7 compute (warpgroup w handles key columns [64w, 64w+64) of the block; in the epilogue,
// head-dim columns [D/2*w, ...)), 8 = TMA producer, 9 = MMA issuer, 10 = TMEM owner, 11 idle
// (setmaxnreg is a warpgroup-wide instruction).
#include <cstdlib>

#include "../fa_common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace fa {

using namespace ptx;

namespace {

constexpr int kB = 128;                 // query rows per item == keys per block
constexpr int kChunkBytes = 128 * 128;  // [128 rows][64 x 16-bit]
constexpr int kThreads = 384;
constexpr int kWarpProducer = 8, kWarpMma = 9, kWarpTmem = 10;
constexpr int kRegsCompute = 200, kRegsOther = 72;

enum DqWait { W_Q_ALIGN = 40, W_Q_QDO = 41, W_Q_KV_FULL = 42, W_Q_KV_EMPTY = 43, W_Q_S = 44, W_Q_DP = 45, W_Q_DS = 46,
              W_Q_DONE = 47, W_Q_QDO_FREE = 48, W_Q_DQ_FREE = 49, W_Q_ITEM = 50 };

template <int DH>
struct QCfg {
  static constexpr int NCHUNK = DH / 64;
  static constexpr int TILE_BYTES = NCHUNK * kChunkBytes;  // one Q / dO / K / V tile
  // K(j) is needed from S(j) (issued a block early) to dQ(j), V(j) only by dP(j): K gets the deeper ring
  static constexpr int NSK = DH > 64 ? 3 : 4;
  static constexpr int NSV = DH > 64 ? 2 : 4;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = TILE_BYTES;
  static constexpr int OFF_K = 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + NSK * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + NSV * TILE_BYTES;
  static constexpr int NBAR = 2 * NSK + 2 * NSV + 14;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 80;  // + tmem address, abort flag, 4 item numbers, 9 read counters
  static constexpr int COL_S = 0, COL_DP = 128, COL_DS = 256, COL_DQ = 384;  // dS: two 64-column buffers
  static constexpr int TMEM_COLS = 512;
};

struct DqTcParams {
  CUtensorMap tq, tk, tv, tdo;
  FaBwdArgs a;
  int n_mblk;   // 128-row query blocks per (batch, head) of the longest sequence
  int n_items;  // n_mblk * heads * batch
  int* next_item;  // work counter, cleared by the host before the launch
};

template <typename T>
struct QFmt;
template <>
struct QFmt<__half> {
  static constexpr int kIdesc = 0;
};
template <>
struct QFmt<__nv_bfloat16> {
  static constexpr int kIdesc = 1;
};

// One work item, decoded the same way by every warp role.
struct Item {
  SeqInfo si;
  int hq, hk, b, m0, n_lo, iters;
  bool live;  // has rows (a packed batch entry may be shorter than the longest sequence)
};
__device__ __forceinline__ Item decode_item(const DqTcParams& P, int item) {
  const FaBwdArgs& a = P.a;
  Item it;
  // Items of one (batch, head) are adjacent, so the CTAs working at the same time stream the same K / V
  // tiles and find them in L2 (148 heads at once would not fit); within a head the heavy query blocks
  // (bottom rows of a causal mask) come first, as longest-first scheduling wants.
  const int bh = item / P.n_mblk, mrank = item - bh * P.n_mblk;
  it.b = bh / a.heads;
  it.hq = bh - it.b * a.heads;
  it.hk = it.hq / (a.heads / a.heads_k);
  it.m0 = (P.n_mblk - 1 - mrank) * kB;
  it.si = seq_info(a.cu_seqlens_q, a.cu_seqlens_k, nullptr, nullptr, a.seqlen_q, a.seqlen_k, a.use_mask_shift, a.mask_shift,
                   it.b);
  it.live = it.m0 < it.si.sq;
  it.n_lo = 0;
  it.iters = 0;
  if (it.live) {
    int n_hi;
    key_block_range(it.m0, kB, kB, it.si.sk, it.si.shift, a.window_left, a.window_right, it.n_lo, n_hi);
    it.iters = n_hi - it.n_lo;
  }
  return it;
}

template <typename T, int DH>
__global__ void __launch_bounds__(kThreads, 1) bwd_dq_tc_kernel(const __grid_constant__ DqTcParams P) {
  using C = QCfg<DH>;
  constexpr int NSK = C::NSK, NSV = C::NSV;
  const FaBwdArgs& a = P.a;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t s_base = smem_addr(smem);
  const uint32_t sQ = s_base + C::OFF_Q, sDO = s_base + C::OFF_DO;
  auto sK = [&](int st) { return s_base + C::OFF_K + st * C::TILE_BYTES; };
  auto sV = [&](int st) { return s_base + C::OFF_V + st * C::TILE_BYTES; };
  const uint32_t bar0 = s_base + C::OFF_BAR;
  auto bar_k_full = [&](int st) { return bar0 + 8 * st; };
  auto bar_k_empty = [&](int st) { return bar0 + 8 * (NSK + st); };
  auto bar_v_full = [&](int st) { return bar0 + 8 * (2 * NSK + st); };
  auto bar_v_empty = [&](int st) { return bar0 + 8 * (2 * NSK + NSV + st); };
  constexpr int kB0 = 2 * NSK + 2 * NSV;
  // per block: S complete / read, dP complete / read, dS written.  per item: Q+dO loaded / free again,
  // dQ complete / read out.
  const uint32_t bar_s = bar0 + 8 * kB0, bar_sread = bar0 + 8 * (kB0 + 1), bar_dp = bar0 + 8 * (kB0 + 2),
                 bar_dpread = bar0 + 8 * (kB0 + 3), bar_ds = bar0 + 8 * (kB0 + 4), bar_qdo = bar0 + 8 * (kB0 + 5),
                 bar_qdo_free = bar0 + 8 * (kB0 + 6), bar_done = bar0 + 8 * (kB0 + 7), bar_dq_free = bar0 + 8 * (kB0 + 8);
  auto bar_item = [&](int n) { return bar0 + 8 * (kB0 + 9 + (n & 3)); };  // item number n has been published
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_BAR + C::NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + C::NBAR * 8 + 4);
  // Items are handed out by a global counter (dynamic, longest first, like the hardware's CTA scheduler).
  // The producer fetches them, one ahead, and publishes the n-th item of this CTA in slot n & 3; the other
  // readers (8 compute warps, the MMA issuer) note how many slots they have read — items without blocks
  // pass through them without any other synchronisation — and a slot is rewritten only after all have
  // read it.  -1 ends the list.
  volatile int* item_ring = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + C::NBAR * 8 + 16);
  volatile int* seen = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + C::NBAR * 8 + 32);  // [0..7] compute warps, [8] MMA

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = g_status;
    for (int i = 0; i < 9; ++i) seen[i] = 0;
    if (s_base & 1023u) {  // the swizzled tiles need a 1024-byte aligned base
      *abort_flag = W_Q_ALIGN;
      atomicCAS(&g_status, 0, (int)W_Q_ALIGN);
    }
    for (int s = 0; s < NSK; ++s) {
      mbar_init(bar_k_full(s), 1);
      mbar_init(bar_k_empty(s), 1);
    }
    for (int s = 0; s < NSV; ++s) {
      mbar_init(bar_v_full(s), 1);
      mbar_init(bar_v_empty(s), 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_sread, 8);
    mbar_init(bar_dp, 1);
    mbar_init(bar_dpread, 8);
    mbar_init(bar_ds, 8);
    mbar_init(bar_qdo, 1);
    mbar_init(bar_qdo_free, 1);
    mbar_init(bar_done, 1);
    mbar_init(bar_dq_free, 8);
    for (int n = 0; n < 4; ++n) mbar_init(bar_item(n), 1);
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
  const bool run = (*abort_flag == 0);
  const float scale_log2 = a.softmax_scale * kLog2e;

  if (warp < 8) {
    // ---------------------------------------------------------------- compute warpgroups
    setmaxnreg_inc<kRegsCompute>();
    const int w = warp >> 2;                    // key-column half / head-dim half
    const int r = (warp & 3) * 32 + lane;       // query row of this thread within the item
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_off + C::COL_S + w * 64;
    const uint32_t tdP = tmem + lane_off + C::COL_DP + w * 64;
    // a wait whose answer is the same in all lanes: the TMEM loads and stores that follow are warp-wide
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, code, abort_flag)) != 0;
    };
    bool ok = run;
    int g = 0;   // blocks done by this CTA: phase of the per-block barriers, dS buffer, K ring position
    int nl = 0;  // items with blocks done by this CTA: phase of the per-item barriers
    for (int n = 0; ok; ++n) {
      ok = wait_all(bar_item(n), (n >> 2) & 1, W_Q_ITEM);
      if (!ok) break;
      const int item = item_ring[n & 3];
      __syncwarp();
      if (lane == 0) seen[warp] = n + 1;
      if (item < 0) break;
      const Item it = decode_item(P, item);
      if (!it.live) continue;
      const SeqInfo& si = it.si;
      const int m0 = it.m0, hq = it.hq, b = it.b;
      const int qrow = m0 + r;
      // per-row statistics of the forward pass; +inf LSE (rows past the end or without keys) gives P = 0
      float lse2 = INFINITY, dsum = 0.f;
      if (qrow < si.sq) {
        lse2 = a.softmax_lse[((int64_t)b * a.heads + hq) * a.lse_seqlen + qrow] * kLog2e;
        dsum = a.softmax_d[((int64_t)b * a.heads + hq) * a.d_seqlen + qrow];
      }
      // keys this row can see: [k_lo, k_hi]
      int k_lo = 0, k_hi = si.sk - 1;
      if (a.window_right >= 0) k_hi = min(k_hi, qrow + si.shift + a.window_right);
      if (a.window_left >= 0) k_lo = max(k_lo, qrow + si.shift - a.window_left);
      for (int j = 0; j < it.iters && ok; ++j, ++g) {
        const int n0 = (it.n_lo + j) * kB;
        const bool need_mask = (n0 + kB > si.sk) ||
                               (a.window_right >= 0 && n0 + kB - 1 > m0 + si.shift + a.window_right) ||
                               (a.window_left >= 0 && n0 < m0 + kB - 1 + si.shift - a.window_left);
        // ---- P = exp2(S * scale - LSE), 64 key columns per thread, kept in registers
        ok = wait_all(bar_s, g & 1, W_Q_S);
        if (!ok) break;
        tc_fence_after();
        float p[64];
        {
          uint32_t s0[32], s1[32];
          tmem_ld32(tS, s0);
          tmem_ld32(tS + 32, s1);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_sread);  // S is in registers: the next S may overwrite it
#pragma unroll
          for (int c = 0; c < 64; ++c)
            p[c] = ex2(fmaf(__uint_as_float(c < 32 ? s0[c & 31] : s1[c & 31]), scale_log2, -lse2));
        }
        if (need_mask) {
          const int c_lo = k_lo - n0 - w * 64, c_hi = k_hi - n0 - w * 64;
#pragma unroll
          for (int c = 0; c < 64; ++c) p[c] = (c >= c_lo && c <= c_hi) ? p[c] : 0.f;
        }
        // ---- dS = P o (dP - D), 16-bit, into this block's dS buffer
        ok = wait_all(bar_dp, g & 1, W_Q_DP);
        if (!ok) break;
        tc_fence_after();
        {
          uint32_t d0[32], d1[32], pk[32];
          tmem_ld32(tdP, d0);
          tmem_ld32(tdP + 32, d1);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_dpread);  // dP is in registers: the next dP may overwrite it
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float x0 = p[c] * (__uint_as_float(c < 32 ? d0[c & 31] : d1[c & 31]) - dsum);
            const float x1 = p[c + 1] * (__uint_as_float(c < 32 ? d0[(c + 1) & 31] : d1[(c + 1) & 31]) - dsum);
            pk[c >> 1] = Pack<T>::two(x0, x1);
          }
          // the buffer held dS of two blocks ago: that block's dQ MMA, whose commit releases its K tile,
          // must have read it (K tile number == block number)
          if (g >= 2) {
            ok = wait_all(bar_k_empty((g - 2) % NSK), ((g - 2) / NSK) & 1, W_Q_KV_EMPTY);
            if (!ok) break;
          }
          tmem_st32(tmem + lane_off + C::COL_DS + (g & 1) * 64 + w * 32, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ds);
      }
      if (!ok) break;
      // ---- the item's dQ * softmax_scale
      if (it.iters > 0) {
        ok = wait_all(bar_done, nl & 1, W_Q_DONE);
        if (!ok) break;
        tc_fence_after();
      }
      {
        const uint32_t tdQ = tmem + lane_off + C::COL_DQ + w * (DH / 2);
        T* gq = reinterpret_cast<T*>(a.dq.ptr) + si.q_batch * a.dq.stride_b + (si.q_row0 + qrow) * a.dq.stride_s +
                (int64_t)hq * a.dq.stride_h;
        const float sc = a.softmax_scale;
#pragma unroll
        for (int c0 = 0; c0 < DH / 2; c0 += 32) {
          uint32_t o[32];
          if (it.iters > 0) {  // uniform for the CTA
            tmem_ld32(tdQ + c0, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
          if (qrow >= si.sq) continue;
          const int col0 = w * (DH / 2) + c0;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (col0 + i < a.head_dim) {
              uint4 v;
              v.x = Pack<T>::two(__uint_as_float(o[i]) * sc, __uint_as_float(o[i + 1]) * sc);
              v.y = Pack<T>::two(__uint_as_float(o[i + 2]) * sc, __uint_as_float(o[i + 3]) * sc);
              v.z = Pack<T>::two(__uint_as_float(o[i + 4]) * sc, __uint_as_float(o[i + 5]) * sc);
              v.w = Pack<T>::two(__uint_as_float(o[i + 6]) * sc, __uint_as_float(o[i + 7]) * sc);
              *reinterpret_cast<uint4*>(gq + col0 + i) = v;
            }
          }
        }
      }
      if (it.iters > 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dq_free);  // the next item may start accumulating its dQ
        ++nl;
      }
    }
  } else {
    setmaxnreg_dec<kRegsOther>();
    if (warp == kWarpProducer) {
      // -------------------------------------------------------------- TMA producer
      if (lane == 0 && run) {
        prefetch_tensormap(&P.tq);
        prefetch_tensormap(&P.tk);
        prefetch_tensormap(&P.tv);
        prefetch_tensormap(&P.tdo);
        bool ok = true;
        int g = 0, nl = 0;  // K / V tiles loaded so far (tile number == block number), items loaded so far
        int item = atomicAdd(P.next_item, 1);
        for (int n = 0; ok; ++n) {
          if (n >= 4) {  // slot n & 3 still holds item n - 4: both readers must be past it
            const long long t0 = clock64();
            auto behind = [&]() {
              int m = seen[8];
              for (int i = 0; i < 8; ++i) m = min(m, seen[i]);
              return m < n - 3;
            };
            while (behind()) {
              if (*abort_flag || clock64() - t0 > kWaitCycles) {
                ok = false;
                break;
              }
            }
            if (!ok) {
              if (*abort_flag == 0) {
                *abort_flag = W_Q_ITEM;
                atomicCAS(&g_status, 0, (int)W_Q_ITEM);
              }
              break;
            }
          }
          item_ring[n & 3] = item < P.n_items ? item : -1;
          mbar_arrive(bar_item(n));  // release: the slot is visible to whoever sees the phase complete
          if (item >= P.n_items) break;
          const int next = atomicAdd(P.next_item, 1);  // fetched one item ahead: its latency hides behind this item's loads
          const Item it = decode_item(P, item);
          item = next;
          if (!it.live || it.iters == 0) continue;
          const int kb = (int)it.si.k_batch, qb = (int)it.si.q_batch;
          if (nl > 0) {  // every MMA that reads the previous item's Q / dO has completed
            ok = mbar_wait(bar_qdo_free, (nl - 1) & 1, W_Q_QDO_FREE, abort_flag);
            if (!ok) break;
          }
          mbar_expect_tx(bar_qdo, 2 * C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c) {
            tma_load_4d(sQ + c * kChunkBytes, &P.tq, bar_qdo, c * 64, (int)it.si.q_row0 + it.m0, it.hq, qb);
            tma_load_4d(sDO + c * kChunkBytes, &P.tdo, bar_qdo, c * 64, (int)it.si.q_row0 + it.m0, it.hq, qb);
          }
          ++nl;
          for (int j = 0; j < it.iters && ok; ++j, ++g) {
            const int ks = g % NSK, vs = g % NSV;
            const int row = (int)it.si.k_row0 + (it.n_lo + j) * kB;
            ok = mbar_wait(bar_k_empty(ks), ((g / NSK) & 1) ^ 1, W_Q_KV_EMPTY, abort_flag);
            if (!ok) break;
            mbar_expect_tx(bar_k_full(ks), C::TILE_BYTES);
            for (int c = 0; c < C::NCHUNK; ++c) tma_load_4d(sK(ks) + c * kChunkBytes, &P.tk, bar_k_full(ks), c * 64, row, it.hk, kb);
            ok = mbar_wait(bar_v_empty(vs), ((g / NSV) & 1) ^ 1, W_Q_KV_EMPTY, abort_flag);
            if (!ok) break;
            mbar_expect_tx(bar_v_full(vs), C::TILE_BYTES);
            for (int c = 0; c < C::NCHUNK; ++c) tma_load_4d(sV(vs) + c * kChunkBytes, &P.tv, bar_v_full(vs), c * 64, row, it.hk, kb);
          }
        }
      }
    } else if (warp == kWarpMma) {
      // -------------------------------------------------------------- MMA issuer
      // Each MMA group is issued as soon as its inputs exist and its output columns are free:
      //   S(j+1) once the compute warps hold S(j) in registers, dP(j+1) once they hold dP(j),
      //   dQ(j) once dS(j) is in its buffer (and, for an item's first block, once the compute warps
      //   have read out the previous item's dQ).
      if (lane == 0 && run) {
        constexpr int F = QFmt<T>::kIdesc;
        constexpr uint32_t idesc_s = make_idesc(kB, kB, F, 0, 0);   // S, dP: K-major x K-major, N = 128 keys
        constexpr uint32_t idesc_dq = make_idesc(kB, DH, F, 0, 1);  // dQ: A in TMEM, B MN-major, N = DH
        // One descriptor is built (Q tile, K-major); every other operand differs from it only in the
        // low word: the address field (+ byte offset >> 4) and, for MN-major reads, the LBO field.
        const uint64_t d_base = smem_desc_sw128(sQ, 16, 1024);
        const uint32_t d_lo = (uint32_t)d_base, d_hi = (uint32_t)(d_base >> 32);
        auto dsc = [&](uint32_t lo_add) { return ((uint64_t)d_hi << 32) | (uint64_t)(d_lo + lo_add); };
        constexpr uint32_t kMn = (uint32_t)((kChunkBytes - 16) >> 4) << 16;  // K-major -> MN-major (LBO = chunk stride)
        constexpr uint32_t oQ = 0, oDO = C::TILE_BYTES >> 4, oK = (C::OFF_K - C::OFF_Q) >> 4, oV = (C::OFF_V - C::OFF_Q) >> 4,
                           kTile16 = C::TILE_BYTES >> 4;
        auto koff = [](int kk) { return (uint32_t)(((kk >> 2) * kChunkBytes + (kk & 3) * 32) >> 4); };  // K-major k-step
        auto moff = [](int kk) { return (uint32_t)((kk * 2048) >> 4) + kMn; };                          // MN-major k-step
        auto issue_s = [&](uint32_t d_col, uint32_t a_lo, uint32_t b_lo, uint32_t bar) {
#pragma unroll
          for (int kk = 0; kk < DH / 16; ++kk) mma_ss(tmem + d_col, dsc(a_lo + koff(kk)), dsc(b_lo + koff(kk)), idesc_s, kk > 0);
          tc_commit(bar);
        };
        bool ok = true;
        int g = 0, nl = 0;
        // ring position and phase of K(g) and of V(g + 1)'s predecessor bookkeeping: tile number == block number
        int ks = 0, vs = 0;            // positions of K(g), V(g)
        uint32_t kph = 0, vph = 0;     // phases of their full barriers
        auto k_next = [&](int& s_, uint32_t& ph_) {
          if (++s_ == NSK) {
            s_ = 0;
            ph_ ^= 1;
          }
        };
        auto v_next = [&](int& s_, uint32_t& ph_) {
          if (++s_ == NSV) {
            s_ = 0;
            ph_ ^= 1;
          }
        };
        for (int n = 0; ok; ++n) {
          ok = mbar_wait(bar_item(n), (n >> 2) & 1, W_Q_ITEM, abort_flag);
          if (!ok) break;
          const int item = item_ring[n & 3];
          seen[8] = n + 1;
          if (item < 0) break;
          const Item it = decode_item(P, item);
          if (!it.live || it.iters == 0) continue;
          ok = mbar_wait(bar_qdo, nl & 1, W_Q_QDO, abort_flag);
          if (ok && g > 0) {  // the last S and dP of the previous item have been read into registers
            ok = mbar_wait(bar_sread, (g - 1) & 1, W_Q_S, abort_flag);
            if (ok) ok = mbar_wait(bar_dpread, (g - 1) & 1, W_Q_DP, abort_flag);
          }
          if (ok) ok = mbar_wait(bar_k_full(ks), kph, W_Q_KV_FULL, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_s(C::COL_S, oQ, oK + ks * kTile16, bar_s);
          ok = mbar_wait(bar_v_full(vs), vph, W_Q_KV_FULL, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_s(C::COL_DP, oDO, oV + vs * kTile16, bar_dp);
          tc_commit(bar_v_empty(vs));
          // Q and dO are last read by the S and dP of the item's last block: released as soon as those are issued
          if (it.iters == 1) tc_commit(bar_qdo_free);
          v_next(vs, vph);  // (vs, vph) now: V(g + 1)
          // barriers of the next group are tested one MMA group ahead of their use (see mbar_test)
          int nks = ks;
          uint32_t nkph = kph;
          k_next(nks, nkph);  // K(g + 1)
          uint32_t h_sread = mbar_test(bar_sread, g & 1), h_k = mbar_test(bar_k_full(nks), nkph), h_dpread = 0, h_v = 0, h_ds = 0;
          for (int j = 0; j < it.iters && ok; ++j, ++g) {
            const bool more = j + 1 < it.iters;
            if (more) {
              ok = mbar_wait_probed(h_sread, bar_sread, g & 1, W_Q_S, abort_flag);
              if (ok) ok = mbar_wait_probed(h_k, bar_k_full(nks), nkph, W_Q_KV_FULL, abort_flag);
              if (!ok) break;
              tc_fence_after();
              h_dpread = mbar_test(bar_dpread, g & 1);
              h_v = mbar_test(bar_v_full(vs), vph);
              issue_s(C::COL_S, oQ, oK + nks * kTile16, bar_s);
              ok = mbar_wait_probed(h_dpread, bar_dpread, g & 1, W_Q_DP, abort_flag);
              if (ok) ok = mbar_wait_probed(h_v, bar_v_full(vs), vph, W_Q_KV_FULL, abort_flag);
              if (!ok) break;
              tc_fence_after();
              h_ds = mbar_test(bar_ds, g & 1);
              issue_s(C::COL_DP, oDO, oV + vs * kTile16, bar_dp);
              tc_commit(bar_v_empty(vs));
              if (j + 2 == it.iters) tc_commit(bar_qdo_free);
              v_next(vs, vph);
            } else {
              h_ds = mbar_test(bar_ds, g & 1);
            }
            ok = mbar_wait_probed(h_ds, bar_ds, g & 1, W_Q_DS, abort_flag);
            if (ok && j == 0 && nl > 0) ok = mbar_wait(bar_dq_free, (nl - 1) & 1, W_Q_DQ_FREE, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int ks_now = ks;
            ks = nks;
            kph = nkph;
            k_next(nks, nkph);  // (ks, kph): K(g + 1); (nks, nkph): K(g + 2)
            if (j + 2 < it.iters) {
              h_sread = mbar_test(bar_sread, (g + 1) & 1);
              h_k = mbar_test(bar_k_full(nks), nkph);
            }
            // dQ += dS K: the two warpgroups' halves of dS are the two 32-column halves of this block's buffer
#pragma unroll
            for (int kk = 0; kk < kB / 16; ++kk)
              mma_ts(tmem + C::COL_DQ, tmem + C::COL_DS + (g & 1) * 64 + kk * 8, dsc(oK + ks_now * kTile16 + moff(kk)), idesc_dq,
                     (j > 0) || kk > 0);
            tc_commit(bar_k_empty(ks_now));
          }
          if (!ok) break;
          tc_commit(bar_done);  // the item's dQ is complete
          ++nl;
        }
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == kWarpTmem) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <typename T, int DH>
int launch_bwd_dq_tc(const FaBwdArgs& a, cudaStream_t st) {
  using C = QCfg<DH>;
  DqTcParams P;
  P.a = a;
  const bool varlen = a.cu_seqlens_q != nullptr;
  const int64_t q_rows = varlen ? a.total_q : a.seqlen_q, k_rows = varlen ? a.total_k : a.seqlen_k;
  const int64_t nb = varlen ? 1 : a.batch;
  if (make_tmap_4d(&P.tq, a.q, a.dtype, q_rows, a.heads, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tdo, a.dout, a.dtype, q_rows, a.heads, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tk, a.k, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tv, a.v, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kB)) return 1;
  auto kern = bwd_dq_tc_kernel<T, DH>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) {
      fa_host::set_error("bwd_dq_tc_kernel: cannot reserve %d bytes of shared memory", C::SMEM_BYTES);
      cudaGetLastError();
      return 2;
    }
    attr_set = true;
  }
  P.n_mblk = (a.seqlen_q + kB - 1) / kB;
  const int64_t items = (int64_t)P.n_mblk * a.heads * a.batch;
  if (items <= 0) return 0;
  if (items >= (1ll << 31)) {
    fa_host::set_error("bwd_dq_tc_kernel: too many work items");
    return 1;
  }
  P.n_items = (int)items;
  // the work counter lives in the first word of the caller's dq_accum workspace (not used otherwise on this path)
  P.next_item = reinterpret_cast<int*>(a.dq_accum);
  if (cudaMemsetAsync(P.next_item, 0, sizeof(int), st) != cudaSuccess) {
    fa_host::set_error("bwd_dq_tc_kernel: clearing the work counter failed: %s", cudaGetErrorString(cudaGetLastError()));
    return 2;
  }
  const int sms = fa_host::sm_count();
  dim3 grid((unsigned)(items < sms ? items : sms));  // one persistent CTA per SM
  kern<<<grid, kThreads, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("bwd_dq_tc_kernel");
}

}  // namespace

int bwd_dq_tc_main(const FaBwdArgs& a, cudaStream_t st) {
  const bool bf = a.dtype == FA_DTYPE_BF16;
  if (a.head_dim <= 64) return bf ? launch_bwd_dq_tc<__nv_bfloat16, 64>(a, st) : launch_bwd_dq_tc<__half, 64>(a, st);
  return bf ? launch_bwd_dq_tc<__nv_bfloat16, 128>(a, st) : launch_bwd_dq_tc<__half, 128>(a, st);
}

int bwd_dq_tc_status(bool clear) {
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) {
    int z = 0;
    cudaMemcpyToSymbol(g_status, &z, sizeof(int));
  }
  return v;
}

}  // namespace fa
