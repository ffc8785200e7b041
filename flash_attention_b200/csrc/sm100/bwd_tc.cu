// Backward attention on tcgen05 tensor cores (head dim <= 128), part 1 of 2: dK and dV.
//
// The backward pass is split in two kernels that each keep their result stationary in tensor memory
// and recompute S and dP: this one (dK, dV; one CTA per 128 keys) and bwd_dq_tc.cu (dQ; one CTA per
// 128 queries).  The single-kernel form of the reference, compute_dq_dk_dv_1colblock
// (csrc/flash_attn/src/flash_bwd_kernel.h:425-1112), adds every block's dQ into an fp32 accumulator
// with atomics; on this GPU an SM sustains only ~26 bytes/clk of fp32 reductions into the L2 (64 KiB
// per block = ~2500 cycles, about the block's whole tensor-core time), and the saturated L2 triples
// the latency of the Q / dO tile loads.  Two more MMAs per block cost less than that, need no
// workspace, and make the gradient deterministic.
//
// One CTA owns 128 keys of one (batch, KV head) and walks every 128-row query block that can see
// them, for every query head of the KV head's group (so grouped-query dK/dV need no expanded
// temporaries or group reduction, cf. flash_api.cpp:744-751, 799-803).  Everything is computed
// TRANSPOSED so that the operands the tensor cores need next are already where tcgen05 wants them:
//   S^T  = K Q^T          (lanes = keys, columns = queries)            SS MMA  -> TMEM tS
//   dP^T = V dO^T                                                       SS MMA  -> TMEM tdP
//   P^T  = exp2(S^T*scale*log2e - LSE*log2e)        one thread per key  -> TMEM (16-bit, over tdP)
//   dS^T = P^T o (dP^T - D)                                             -> TMEM (16-bit, over tdP)
//   dV  += P^T  dO        A = P^T from TMEM, B = dO tile (MN-major)     -> TMEM tdV
//   dK  += dS^T Q         A = dS^T from TMEM, B = Q tile (MN-major)      -> TMEM tdK
//
// Warps: 0-7 compute (warpgroup w handles query columns [64w, 64w+64) of the block; in the
// epilogue, head-dim columns [D/2*w, ...)), 8 = TMA producer, 9 = MMA issuer, 10 = loader of the
// per-row LSE / D vectors and TMEM owner, 11 idle (setmaxnreg is a warpgroup-wide instruction).
#include <cstdlib>

#include "../fa_common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace fa {

using namespace ptx;

StatusRef status_ref(bool may_allocate);

namespace {

constexpr int kB = 128;                 // query rows per block == keys per CTA
constexpr int kChunkBytes = 128 * 128;  // [128 rows][64 x 16-bit]

constexpr int kThreads = 384;
constexpr int kWarpProducer = 8, kWarpMma = 9, kWarpStats = 10, kWarpMmaS = 11;
constexpr int kRegsCompute = 200, kRegsOther = 72;

enum BwdWait { W_B_KV = 21, W_B_QDO_FULL = 22, W_B_QDO_EMPTY = 23, W_B_STATS_FULL = 24, W_B_STATS_EMPTY = 25,
               W_B_S = 26, W_B_DP = 27, W_B_PDS = 28, W_B_ALIGN = 20 };

template <int DH>
struct BCfg {
  static constexpr int NCHUNK = DH / 64;
  static constexpr int TILE_BYTES = NCHUNK * kChunkBytes;  // one Q / dO / K / V tile
  // Q(i) is needed from S^T(i) (issued a block early) to dK(i), dO(i) from dP^T(i) to dV(i): Q gets the deeper ring
  static constexpr int NSQ = 3, NSO = 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE_BYTES;
  static constexpr int OFF_Q = 2 * TILE_BYTES;
  static constexpr int OFF_DO = OFF_Q + NSQ * TILE_BYTES;
  static constexpr int OFF_STATS = OFF_DO + NSO * TILE_BYTES;  // 2 slots x (128 lse2, 128 dsum) fp32
  static constexpr int OFF_BAR = OFF_STATS + 2 * 1024;
  static constexpr int NBAR = 24;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 32;
  static constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + DH;
  static constexpr int TMEM_COLS = 512;
};

struct BwdTcParams {
  CUtensorMap tq, tk, tv, tdo;
  FaBwdArgs a;
  StatusRef status;
};

template <typename T>
struct BFmt;
template <>
struct BFmt<__half> {
  static constexpr int kIdesc = 0;
};
template <>
struct BFmt<__nv_bfloat16> {
  static constexpr int kIdesc = 1;
};


template <typename T, int DH>
__global__ void __launch_bounds__(kThreads, 1) bwd_tc_kernel(const __grid_constant__ BwdTcParams P) {
  using C = BCfg<DH>;
  const FaBwdArgs& a = P.a;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t s_base = smem_addr(smem);
  constexpr int NSQ = C::NSQ, NSO = C::NSO;
  const uint32_t sK = s_base + C::OFF_K, sV = s_base + C::OFF_V;
  auto sQ = [&](int slot) { return s_base + C::OFF_Q + slot * C::TILE_BYTES; };
  auto sDO = [&](int slot) { return s_base + C::OFF_DO + slot * C::TILE_BYTES; };
  float* sStats = reinterpret_cast<float*>(smem + C::OFF_STATS);
  const uint32_t bar0 = s_base + C::OFF_BAR;
  const uint32_t bar_kv = bar0;
  auto bar_q_full = [&](int s) { return bar0 + 8 * (1 + s); };
  auto bar_q_empty = [&](int s) { return bar0 + 8 * (4 + s); };
  auto bar_do_full = [&](int s) { return bar0 + 8 * (7 + s); };
  auto bar_do_empty = [&](int s) { return bar0 + 8 * (9 + s); };
  auto bar_st_full = [&](int s) { return bar0 + 8 * (11 + s); };
  auto bar_st_empty = [&](int s) { return bar0 + 8 * (13 + s); };
  const uint32_t bar_s = bar0 + 8 * 15, bar_dp = bar0 + 8 * 16, bar_ds = bar0 + 8 * 17, bar_p = bar0 + 8 * 18,
                 bar_sread = bar0 + 8 * 19;
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_BAR + C::NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + C::NBAR * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = a.heads / a.heads_k;
  const SeqInfo si = seq_info(a.cu_seqlens_q, a.cu_seqlens_k, nullptr, nullptr, a.seqlen_q, a.seqlen_k,
                              a.use_mask_shift, a.mask_shift, b);
  const int n0 = nblk * kB;
  if (n0 >= si.sk) return;
  int m_lo, m_hi;
  query_block_range(n0, kB, kB, si.sq, si.shift, a.window_left, a.window_right, m_lo, m_hi);
  const int nmb = m_hi - m_lo;
  const int iters = nmb * group;

  if (threadIdx.x == 0) {
    abort_init(abort_flag, P.status);
    if (s_base & 1023u) abort_raise(abort_flag, W_B_ALIGN);  // the swizzled tiles need a 1024-byte aligned base
    mbar_init(bar_kv, 1);
    for (int s = 0; s < NSQ; ++s) {
      mbar_init(bar_q_full(s), 1);
      mbar_init(bar_q_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_do_full(s), 1);
      mbar_init(bar_do_empty(s), 1);
      mbar_init(bar_st_full(s), 1);
      mbar_init(bar_st_empty(s), 8);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_dp, 1);
    mbar_init(bar_ds, 8);
    mbar_init(bar_p, 8);
    mbar_init(bar_sread, 8);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == kWarpStats) {
    tmem_alloc(smem_addr(const_cast<uint32_t*>(tmem_ptr_smem)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;
  const bool run = (*abort_flag == 0) && iters > 0;

  const float scale_log2 = a.softmax_scale * kLog2e;
  // (query head, query block) of iteration `it`, stepped without divisions: blocks m_lo..m_hi-1 of one head, then the next head
  struct Walk {
    int mb, hq, lo, hi;
    __device__ void next() {
      if (++mb == hi) {
        mb = lo;
        ++hq;
      }
    }
  };
  const Walk walk0{m_lo, hk * group, m_lo, m_hi};

  if (warp < 8) {
    // ---------------------------------------------------------------- compute warpgroups
    setmaxnreg_inc<kRegsCompute>();
    const int w = warp >> 2;                       // query-column half / head-dim half
    const int kr = (warp & 3) * 32 + lane;         // key row of this thread within the CTA tile
    const int key = n0 + kr;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_off + C::COL_S, tdP = tmem + lane_off + C::COL_DP;
    bool ok = (*abort_flag == 0);  // with iters == 0 the loop is skipped and the epilogue writes zeros
    Walk wk = walk0;
    for (int it = 0; it < iters && ok; ++it, wk.next()) {
      const int slot = it & 1, par = (it >> 1) & 1;
      const int m0 = wk.mb * kB;
      // per-thread visible query columns [c_lo, c_hi] of this block (c = query row - m0)
      int c_lo = 0, c_hi = min(kB, si.sq - m0) - 1;
      if (a.window_right >= 0) c_lo = max(c_lo, key - si.shift - a.window_right - m0);
      if (a.window_left >= 0) c_hi = min(c_hi, key - si.shift + a.window_left - m0);
      if (key >= si.sk) c_hi = -1;
      const bool need_mask = (n0 + kB > si.sk) || (m0 + kB > si.sq) ||
                             (a.window_right >= 0 && n0 + kB - 1 > m0 + si.shift + a.window_right) ||
                             (a.window_left >= 0 && n0 < m0 + kB - 1 + si.shift - a.window_left);
      // ---- P^T = exp2(S^T * scale - LSE), 64 query columns per thread, into TMEM as the A operand of dV
      ok = mbar_wait(bar_s, it & 1, W_B_S, abort_flag);
      if (!ok) break;
      const float* lse2 = sStats + slot * 256 + w * 64;
      const float* dsum = sStats + slot * 256 + 128 + w * 64;
      ok = mbar_wait(bar_st_full(slot), par, W_B_STATS_FULL, abort_flag);
      if (!ok) break;
      tc_fence_after();
      float p[64];
      {
        uint32_t s0[32], s1[32];
        tmem_ld32(tS + w * 64, s0);
        tmem_ld32(tS + w * 64 + 32, s1);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sread);  // S^T(it) is in registers: the next S^T may overwrite it
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 l4 = reinterpret_cast<const float4*>(lse2)[c4];
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c4 * 4 + e;
            p[c] = ex2(fmaf(__uint_as_float(c < 32 ? s0[c & 31] : s1[c & 31]), scale_log2, -lv[e]));
          }
        }
      }
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int cc = w * 64 + c;
          p[c] = (cc >= c_lo && cc <= c_hi) ? p[c] : 0.f;
        }
      }
      // ---- dP^T(it) into registers, then P^T (16-bit) over the first half of this warpgroup's dP^T
      //      columns, where it is the A operand of dV
      ok = mbar_wait(bar_dp, it & 1, W_B_DP, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t d0[32], d1[32];
      tmem_ld32(tdP + w * 64, d0);
      tmem_ld32(tdP + w * 64 + 32, d1);
      tmem_wait_ld();
      {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) pk[c >> 1] = Pack<T>::two(p[c], p[c + 1]);
        tmem_st32(tdP + w * 64, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      // ---- dS^T = P^T o (dP^T - D), 16-bit, over the second half of this warpgroup's dP^T columns,
      //      where it is the A operand of dK
      {
        uint32_t dk[32];
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 d4 = reinterpret_cast<const float4*>(dsum)[c4];
          const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int e = 0; e < 4; e += 2) {
            const int c = c4 * 4 + e;
            const float x0 = p[c] * (__uint_as_float(c < 32 ? d0[c & 31] : d1[c & 31]) - dv[e]);
            const float x1 = p[c + 1] * (__uint_as_float(c < 32 ? d0[(c + 1) & 31] : d1[(c + 1) & 31]) - dv[e + 1]);
            dk[c >> 1] = Pack<T>::two(x0, x1);
          }
        }
        tmem_st32(tdP + w * 64 + 32, dk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_st_empty(slot));
        mbar_arrive(bar_ds);
      }
    }
    // every MMA of the CTA has completed once the last block's Q slot has been released
    if (ok && iters > 0) ok = mbar_wait(bar_q_empty((iters - 1) % NSQ), ((iters - 1) / NSQ) & 1, W_B_QDO_EMPTY, abort_flag);
    tc_fence_after();

    // ---- epilogue: dK (scaled) and dV
    if (ok && *abort_flag == 0) {
      const uint32_t tdV = tmem + lane_off + C::COL_DV, tdK = tmem + lane_off + C::COL_DK;
      const bool valid = key < si.sk;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which ? tdK : tdV;
        const float sc = which ? a.softmax_scale : 1.f;
#pragma unroll
        for (int c0 = 0; c0 < DH / 2; c0 += 32) {
          uint32_t o[32];
          if (iters > 0) {
            tmem_ld32(src + w * (DH / 2) + c0, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
          if (!valid) continue;
          const int col0 = w * (DH / 2) + c0;
          if (a.accumulate_dkv) {
            float* acc = (which ? a.dk_accum : a.dv_accum) +
                         (((int64_t)si.k_batch * a.seqlen_k + si.k_row0 + key) * a.heads_k + hk) * a.head_dim;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (col0 + i < a.head_dim) {
                float4 cur = *reinterpret_cast<float4*>(acc + col0 + i);
                cur.x += __uint_as_float(o[i]) * sc;
                cur.y += __uint_as_float(o[i + 1]) * sc;
                cur.z += __uint_as_float(o[i + 2]) * sc;
                cur.w += __uint_as_float(o[i + 3]) * sc;
                *reinterpret_cast<float4*>(acc + col0 + i) = cur;
              }
            }
          } else {
            const FaTensor& tt = which ? a.dk : a.dv;
            T* g = reinterpret_cast<T*>(tt.ptr) + si.k_batch * tt.stride_b + (si.k_row0 + key) * tt.stride_s + (int64_t)hk * tt.stride_h;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i < a.head_dim) {
                uint4 v;
                v.x = Pack<T>::two(__uint_as_float(o[i]) * sc, __uint_as_float(o[i + 1]) * sc);
                v.y = Pack<T>::two(__uint_as_float(o[i + 2]) * sc, __uint_as_float(o[i + 3]) * sc);
                v.z = Pack<T>::two(__uint_as_float(o[i + 4]) * sc, __uint_as_float(o[i + 5]) * sc);
                v.w = Pack<T>::two(__uint_as_float(o[i + 6]) * sc, __uint_as_float(o[i + 7]) * sc);
                *reinterpret_cast<uint4*>(g + col0 + i) = v;
              }
            }
          }
        }
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
        const int kb = (int)si.k_batch, qb = (int)si.q_batch;
        mbar_expect_tx(bar_kv, 2 * C::TILE_BYTES);
        for (int c = 0; c < C::NCHUNK; ++c) {
          tma_load_4d(sK + c * kChunkBytes, &P.tk, bar_kv, c * 64, (int)si.k_row0 + n0, hk, kb);
          tma_load_4d(sV + c * kChunkBytes, &P.tv, bar_kv, c * 64, (int)si.k_row0 + n0, hk, kb);
        }
        bool ok = true;
        Walk wk = walk0;
        for (int it = 0; it < iters && ok; ++it, wk.next()) {
          const int qs = it % NSQ, os = it % NSO;
          const int row = (int)si.q_row0 + wk.mb * kB, hq = wk.hq;
          ok = mbar_wait(bar_q_empty(qs), ((it / NSQ) & 1) ^ 1, W_B_QDO_EMPTY, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bar_q_full(qs), C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c) tma_load_4d(sQ(qs) + c * kChunkBytes, &P.tq, bar_q_full(qs), c * 64, row, hq, qb);
          ok = mbar_wait(bar_do_empty(os), ((it / NSO) & 1) ^ 1, W_B_QDO_EMPTY, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bar_do_full(os), C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c) tma_load_4d(sDO(os) + c * kChunkBytes, &P.tdo, bar_do_full(os), c * 64, row, hq, qb);
        }
      }
    } else if (warp == kWarpStats) {
      // -------------------------------------------------------------- LSE / D loader
      // The values of the next block are fetched into registers before the wait for a free slot,
      // so that the global-memory latency is not part of the hand-over.
      bool ok = run;
      float l[4], d[4];
      Walk wk = walk0;
      auto fetch = [&]() {
        const int m0 = wk.mb * kB, hq = wk.hq;
        const float* lse_g = a.softmax_lse + ((int64_t)b * a.heads + hq) * a.lse_seqlen;
        const float* d_g = a.softmax_d + ((int64_t)b * a.heads + hq) * a.d_seqlen;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int q = m0 + i * 32 + lane;
          l[i] = q < si.sq ? lse_g[q] : INFINITY;
          d[i] = q < si.sq ? d_g[q] : 0.f;
        }
      };
      if (ok) fetch();
      for (int it = 0; it < iters && ok; ++it) {
        const int slot = it & 1, round = it >> 1;
        ok = mbar_wait(bar_st_empty(slot), (round & 1) ^ 1, W_B_STATS_EMPTY, abort_flag);
        if (!ok) break;
        float* dst = sStats + slot * 256;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dst[i * 32 + lane] = l[i] * kLog2e;  // +inf stays +inf: exp2(x - inf) = 0 for rows without keys / past the end
          dst[128 + i * 32 + lane] = d[i];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_st_full(slot));
        if (it + 1 < iters) {
          wk.next();
          fetch();
        }
      }
    } else if (warp == kWarpMma || warp == kWarpMmaS) {
      // -------------------------------------------------------------- MMA issuer
      // Two issuing threads.  Warp 11 issues S^T(i+1) as soon as the compute warps hold S^T(i) in registers.  Warp 9
      // issues the chain dV(i) | dK(i) | dP^T(i+1): dV(i) waits for P^T(i), dK(i) for dS^T(i); both sit over dP^T(i),
      // and the MMAs of one thread execute in order, so dP^T(i+1) overwrites them only after they were read.
      // MMAs of the two threads are not ordered among themselves and need not be.
      if (run) {  // the whole warp runs the loops (see mma_ss_w); one elected lane issues
        constexpr int F = BFmt<T>::kIdesc;
        constexpr uint32_t idesc_st = make_idesc(kB, kB, F, 0, 0);   // S^T, dP^T: K-major x K-major, N = 128 queries
        constexpr uint32_t idesc_dv = make_idesc(kB, DH, F, 0, 1);   // dV, dK: A K-major (or TMEM), B MN-major, N = DH
        // One descriptor is built (K tile, K-major); every other operand differs from it only in the
        // low word: the address field (+ byte offset >> 4) and, for MN-major reads, the LBO field.
        const uint64_t d_base = smem_desc_sw128(sK, 16, 1024);
        const uint32_t d_lo = (uint32_t)d_base, d_hi = (uint32_t)(d_base >> 32);
        auto dsc = [&](uint32_t lo_add) { return ((uint64_t)d_hi << 32) | (uint64_t)(d_lo + lo_add); };
        constexpr uint32_t kMn = (uint32_t)((kChunkBytes - 16) >> 4) << 16;  // K-major -> MN-major (LBO = chunk stride)
        constexpr uint32_t oK = 0, oV = (C::OFF_V - C::OFF_K) >> 4, oQ = (C::OFF_Q - C::OFF_K) >> 4,
                           oDO = (C::OFF_DO - C::OFF_K) >> 4, kTile16 = C::TILE_BYTES >> 4;
        auto koff = [](int kk) { return (uint32_t)(((kk >> 2) * kChunkBytes + (kk & 3) * 32) >> 4); };  // K-major k-step
        auto moff = [](int kk) { return (uint32_t)((kk * 2048) >> 4) + kMn; };                          // MN-major k-step
        auto issue_st = [&](uint32_t d_col, uint32_t a_lo, uint32_t b_lo, uint32_t bar) {
#pragma unroll
          for (int kk = 0; kk < DH / 16; ++kk) mma_ss_w(tmem + d_col, dsc(a_lo + koff(kk)), dsc(b_lo + koff(kk)), idesc_st, kk > 0);
          tc_commit_w(bar);
        };
        bool ok = mbar_wait_w(bar_kv, 0, W_B_KV, abort_flag);
        if (warp == kWarpMmaS) {
          for (int it = 0; it < iters && ok; ++it) {
            const int qs = it % NSQ;
            if (it > 0) ok = mbar_wait_w(bar_sread, (it - 1) & 1, W_B_S, abort_flag);
            if (ok) ok = mbar_wait_w(bar_q_full(qs), (it / NSQ) & 1, W_B_QDO_FULL, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_st(C::COL_S, oK, oQ + qs * kTile16, bar_s);
          }
        } else {
          if (ok) ok = mbar_wait_w(bar_do_full(0), 0, W_B_QDO_FULL, abort_flag);
          if (ok) {
            tc_fence_after();
            issue_st(C::COL_DP, oV, oDO, bar_dp);
          }
          for (int it = 0; it < iters && ok; ++it) {
            const bool more = it + 1 < iters;
            const int qs = it % NSQ, os = it % NSO, nos = (it + 1) % NSO;
            // P^T(it) is in TMEM over dP^T(it): dV += P^T dO (the warpgroups' halves sit at columns 0 and 64 of
            // the dP^T range); that was the last use of this dO tile
            ok = mbar_wait_w(bar_p, it & 1, W_B_PDS, abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kB / 16; ++kk)
              mma_ts_w(tmem + C::COL_DV, tmem + C::COL_DP + (kk >> 2) * 64 + (kk & 3) * 8, dsc(oDO + os * kTile16 + moff(kk)),
                     idesc_dv, (it > 0) || kk > 0);
            tc_commit_w(bar_do_empty(os));
            // dS^T(it) is in TMEM next to P^T(it) (columns 32 and 96 of the dP^T range): dK += dS^T Q, the last
            // use of this Q tile (S^T(it) of the other issuer read it too: P^T(it) was computed from it)
            ok = mbar_wait_w(bar_ds, it & 1, W_B_PDS, abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kB / 16; ++kk)
              mma_ts_w(tmem + C::COL_DK, tmem + C::COL_DP + 32 + (kk >> 2) * 64 + (kk & 3) * 8, dsc(oQ + qs * kTile16 + moff(kk)),
                     idesc_dv, (it > 0) || kk > 0);
            tc_commit_w(bar_q_empty(qs));
            if (more) {
              ok = mbar_wait_w(bar_do_full(nos), ((it + 1) / NSO) & 1, W_B_QDO_FULL, abort_flag);
              if (!ok) break;
              tc_fence_after();
              issue_st(C::COL_DP, oV, oDO + nos * kTile16, bar_dp);
            }
          }
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
  if (warp == kWarpStats) tmem_dealloc(tmem, C::TMEM_COLS);
}


template <typename T, int DH>
int launch_bwd_tc(const FaBwdArgs& a, cudaStream_t st) {
  using C = BCfg<DH>;
  BwdTcParams P;
  P.a = a;
  const bool varlen = a.cu_seqlens_q != nullptr;
  const int64_t q_rows = varlen ? a.total_q : a.seqlen_q, k_rows = varlen ? a.total_k : a.seqlen_k;
  const int64_t nb = varlen ? 1 : a.batch;
  if (make_tmap_4d(&P.tq, a.q, a.dtype, q_rows, a.heads, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tdo, a.dout, a.dtype, q_rows, a.heads, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tk, a.k, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tv, a.v, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kB)) return 1;
  auto kern = bwd_tc_kernel<T, DH>;
  P.status = status_ref(true);
  static fa_host::DeviceOnce once;
  if (int rc = fa_host::raise_smem_limit(once, reinterpret_cast<const void*>(kern), C::SMEM_BYTES, "bwd_tc_kernel")) return rc;
  dim3 grid((a.seqlen_k + kB - 1) / kB, a.heads_k, a.batch);
  kern<<<grid, kThreads, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("bwd_tc_kernel");
}

}  // namespace

bool bwd_tc_eligible(const FaBwdArgs& a) {
  if (a.head_dim > 256 || a.p_dropout > 0.f) return false;  // head dims 129..256 run in bwd_wide_tc.cu
  if (a.seqlen_k <= 0 || a.seqlen_q <= 0) return false;
  if (!tma_compatible(a.q) || !tma_compatible(a.k) || !tma_compatible(a.v) || !tma_compatible(a.dout)) return false;
  // the epilogues store 16 bytes at a time
  if (!tma_compatible(a.dq)) return false;
  if (!a.accumulate_dkv && (!tma_compatible(a.dk) || !tma_compatible(a.dv))) return false;
  if (a.head_dim % 8) return false;
  if (a.cu_seqlens_q && (a.total_q <= 0 || a.total_k <= 0)) return false;
  return encode_tiled_fn() != nullptr;
}

int bwd_tc_main(const FaBwdArgs& a, cudaStream_t st) {
  const bool bf = a.dtype == FA_DTYPE_BF16;
  if (a.head_dim <= 64) return bf ? launch_bwd_tc<__nv_bfloat16, 64>(a, st) : launch_bwd_tc<__half, 64>(a, st);
  return bf ? launch_bwd_tc<__nv_bfloat16, 128>(a, st) : launch_bwd_tc<__half, 128>(a, st);
}

}  // namespace fa
