// Backward attention main loop on tcgen05 tensor cores (head dim <= 128).
//
// One CTA owns 128 keys of one (batch, KV head) and walks every 128-row query block that can see
// them, for every query head of the KV head's group (so grouped-query dK/dV need no expanded
// temporaries or group reduction, cf. flash_api.cpp:744-751, 799-803, and stay free of atomics).
// Same math as compute_dq_dk_dv_1colblock (csrc/flash_attn/src/flash_bwd_kernel.h:425-1112), but
// everything is computed TRANSPOSED so that the operands the tensor cores need next are already
// where tcgen05 wants them:
//   S^T  = K Q^T          (lanes = keys, columns = queries)            SS MMA  -> TMEM tS
//   dP^T = V dO^T                                                       SS MMA  -> TMEM tdP
//   P^T  = exp2(S^T*scale*log2e - LSE*log2e)        one thread per key  -> TMEM (16-bit, over tS)
//   dS^T = P^T o (dP^T - D)                                             -> shared, [key][query]
//   dV  += P^T  dO        A = P^T from TMEM, B = dO tile (MN-major)     -> TMEM tdV
//   dK  += dS^T Q         A = dS^T from shared (K-major), B = Q tile    -> TMEM tdK
//   dQ   = dS   K         A = the same dS^T bytes read MN-major, B = K  -> TMEM (over tdP)
// dQ leaves TMEM through registers into the shared-memory slot of the block's (already consumed)
// Q / dO tiles and from there, one bulk fp32 add-reduction of 8 KiB per warp, into a BLOCKED dq_accum
// workspace (fa_common.cuh: dq_blocked_offset) that the host cleared; bwd_convert_dq_blocked_kernel
// scales and casts it (generic_bwd.cu).  Scattered 16-byte red.global reductions were measured at
// 37 % of the kernel's time; the bulk form adds whole lines at the memory side.
//
// Warps: 0-7 compute (warpgroup w handles query columns [64w, 64w+64) of the block; at the drain
// and in the epilogue, head-dim columns [D/2*w, ...)), 8 = TMA producer, 9 = MMA issuer,
// 10 = loader of the per-row LSE / D vectors, 11 = TMEM owner.
#include <cstdlib>

#include "../fa_common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace fa {

using namespace ptx;

namespace {

constexpr int kB = 128;                 // query rows per block == keys per CTA
constexpr int kChunkBytes = 128 * 128;  // [128 rows][64 x 16-bit]

enum BwdWait { W_B_KV = 21, W_B_QDO_FULL = 22, W_B_QDO_EMPTY = 23, W_B_STATS_FULL = 24, W_B_STATS_EMPTY = 25,
               W_B_S = 26, W_B_DP = 27, W_B_PDS = 28, W_B_DQ_FULL = 29, W_B_DQ_EMPTY = 30, W_B_ALIGN = 20 };

template <int DH>
struct BCfg {
  static constexpr int NCHUNK = DH / 64;
  static constexpr int TILE_BYTES = NCHUNK * kChunkBytes;  // one Q / dO / K / V tile
  static constexpr int DS_BYTES = 2 * kChunkBytes;         // dS^T: 128 keys x 128 queries x 16-bit
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE_BYTES;
  static constexpr int OFF_QDO = 2 * TILE_BYTES;           // 2 slots x (Q, dO)
  static constexpr int OFF_DS = OFF_QDO + 4 * TILE_BYTES;
  static constexpr int OFF_STATS = OFF_DS + DS_BYTES;      // 2 slots x (128 lse2, 128 dsum) fp32
  static constexpr int OFF_BAR = OFF_STATS + 2 * 1024;
  static constexpr int NBAR = 16;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 16;
  static constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + DH;
  static constexpr int TMEM_COLS = 512;
};

struct BwdTcParams {
  CUtensorMap tq, tk, tv, tdo;
  FaBwdArgs a;
  int debug;      // timing experiments only (FA_B200_DEBUG_BWD); 0 in normal use
  int dq_blocks;  // 128-row blocks per (batch, head) [packed input: per head] of the blocked dq_accum
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
__global__ void __launch_bounds__(384, 1) bwd_tc_kernel(const __grid_constant__ BwdTcParams P) {
  using C = BCfg<DH>;
  const FaBwdArgs& a = P.a;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t s_base = smem_addr(smem);
  const uint32_t sK = s_base + C::OFF_K, sV = s_base + C::OFF_V, sDS = s_base + C::OFF_DS;
  auto sQ = [&](int slot) { return s_base + C::OFF_QDO + slot * 2 * C::TILE_BYTES; };
  auto sDO = [&](int slot) { return s_base + C::OFF_QDO + slot * 2 * C::TILE_BYTES + C::TILE_BYTES; };
  float* sStats = reinterpret_cast<float*>(smem + C::OFF_STATS);
  const uint32_t bar0 = s_base + C::OFF_BAR;
  const uint32_t bar_kv = bar0;
  auto bar_qdo_full = [&](int s) { return bar0 + 8 * (1 + s); };
  auto bar_qdo_empty = [&](int s) { return bar0 + 8 * (3 + s); };
  auto bar_st_full = [&](int s) { return bar0 + 8 * (5 + s); };
  auto bar_st_empty = [&](int s) { return bar0 + 8 * (7 + s); };
  const uint32_t bar_s = bar0 + 8 * 9, bar_dp = bar0 + 8 * 10, bar_pds = bar0 + 8 * 11, bar_dq_full = bar0 + 8 * 12,
                 bar_dq_empty = bar0 + 8 * 13, bar_sread = bar0 + 8 * 14;
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
    *abort_flag = g_status;
    if (s_base & 1023u) {  // the swizzled tiles need a 1024-byte aligned base
      *abort_flag = W_B_ALIGN;
      atomicCAS(&g_status, 0, (int)W_B_ALIGN);
    }
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qdo_full(s), 1);
      mbar_init(bar_qdo_empty(s), 9);  // the MMA commit + 8 warps that staged their dQ piece in the slot
      mbar_init(bar_st_full(s), 1);
      mbar_init(bar_st_empty(s), 8);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_dp, 1);
    mbar_init(bar_pds, 8);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_empty, 8);
    mbar_init(bar_sread, 8);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 11) {
    tmem_alloc(smem_addr(const_cast<uint32_t*>(tmem_ptr_smem)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;
  const bool run = (*abort_flag == 0) && iters > 0;

  const float scale_log2 = a.softmax_scale * kLog2e;
  auto head_of = [&](int it) { return hk * group + it / nmb; };
  auto mblk_of = [&](int it) { return m_lo + it % nmb; };

  if (warp < 8) {
    // ---------------------------------------------------------------- compute warpgroups
    setmaxnreg_inc<200>();
    const int w = warp >> 2;                       // query-column half / head-dim half
    const int kr = (warp & 3) * 32 + lane;         // key row of this thread within the CTA tile
    const int key = n0 + kr;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_off + C::COL_S, tdP = tmem + lane_off + C::COL_DP;
    bool ok = (*abort_flag == 0);  // with iters == 0 the loop is skipped and the epilogue writes zeros
    for (int it = 0; it < iters && ok; ++it) {
      const int slot = it & 1, par = (it >> 1) & 1;
      const int m0 = mblk_of(it) * kB;
      const int hq = head_of(it);
      // per-thread visible query columns [c_lo, c_hi] of this block (c = query row - m0)
      int c_lo = 0, c_hi = min(kB, si.sq - m0) - 1;
      if (a.window_right >= 0) c_lo = max(c_lo, key - si.shift - a.window_right - m0);
      if (a.window_left >= 0) c_hi = min(c_hi, key - si.shift + a.window_left - m0);
      if (key >= si.sk) c_hi = -1;
      const bool need_mask = (n0 + kB > si.sk) || (m0 + kB > si.sq) ||
                             (a.window_right >= 0 && n0 + kB - 1 > m0 + si.shift + a.window_right) ||
                             (a.window_left >= 0 && n0 < m0 + kB - 1 + si.shift - a.window_left);
      ok = mbar_wait(bar_st_full(slot), par, W_B_STATS_FULL, abort_flag);
      if (!ok) break;
      const float* lse2 = sStats + slot * 256 + w * 64;
      const float* dsum = sStats + slot * 256 + 128 + w * 64;
      ok = mbar_wait(bar_s, it & 1, W_B_S, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t su[2][32];
      tmem_ld32(tS + w * 64, su[0]);
      tmem_ld32(tS + w * 64 + 32, su[1]);
      tmem_wait_ld();
      float p[64];
#pragma unroll
      for (int c4 = 0; c4 < 16; ++c4) {
        const float4 l4 = reinterpret_cast<const float4*>(lse2)[c4];
        const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = c4 * 4 + e;
          float x = (P.debug & 4) ? __uint_as_float(su[c >> 5][c & 31]) * 1e-3f
                                  : fast_exp2(fmaf(__uint_as_float(su[c >> 5][c & 31]), scale_log2, -lv[e]));
          if (need_mask) {
            const int cc = w * 64 + c;
            x = (cc >= c_lo && cc <= c_hi) ? x : 0.f;
          }
          p[c] = x;
        }
      }
      // both warpgroups must have read S^T before P^T is written over its columns (a bounded
      // mbarrier rendezvous rather than bar.sync, so that an aborting kernel cannot strand a warp)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sread);
      ok = mbar_wait(bar_sread, it & 1, W_B_S, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) pk[c >> 1] = Pack<T>::two(p[c], p[c + 1]);
        tmem_st32(tS + w * 32, pk);
      }
      ok = mbar_wait(bar_dp, it & 1, W_B_DP, abort_flag);
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(tdP + w * 64, su[0]);
      tmem_ld32(tdP + w * 64 + 32, su[1]);
      tmem_wait_ld();
      {
        unsigned char* ds_row = smem + C::OFF_DS + w * kChunkBytes + kr * 128;
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {
          const float4 da = reinterpret_cast<const float4*>(dsum)[c16 * 2], db = reinterpret_cast<const float4*>(dsum)[c16 * 2 + 1];
          const float dv8[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
          uint32_t vv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c16 * 8 + e * 2;
            const float d0 = p[c] * (__uint_as_float(su[c >> 5][c & 31]) - dv8[e * 2]);
            const float d1 = p[c + 1] * (__uint_as_float(su[(c + 1) >> 5][(c + 1) & 31]) - dv8[e * 2 + 1]);
            vv[e] = Pack<T>::two(d0, d1);
          }
          *reinterpret_cast<uint4*>(ds_row + (((c16 ^ kr) & 7) << 4)) = make_uint4(vv[0], vv[1], vv[2], vv[3]);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      fence_proxy_async();  // dS^T was written with ordinary stores and is read by the tensor core
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_st_empty(slot));
        mbar_arrive(bar_pds);
      }
      // ---- drain dQ of this block: lanes are query rows now, this warpgroup takes DH/2 columns
      ok = mbar_wait(bar_dq_full, it & 1, W_B_DQ_FULL, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        // TMEM -> registers; the dP^T/dQ columns are free again as soon as the loads have landed
        uint32_t o[DH / 64][32];
#pragma unroll
        for (int j = 0; j < DH / 64; ++j) tmem_ld32(tdP + w * (DH / 2) + j * 32, o[j]);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dq_empty);
        // registers -> shared staging (the Q / dO tile of this block, which no MMA reads any more), laid out
        // exactly like the warp's 32-row piece of the blocked dq_accum: [4-column chunk][row][4 floats]
        constexpr int kWarpBytes = 32 * (DH / 2) * 4;
        unsigned char* stage = smem + C::OFF_QDO + slot * 2 * C::TILE_BYTES + w * C::TILE_BYTES + (warp & 3) * kWarpBytes;
#pragma unroll
        for (int c4 = 0; c4 < DH / 8; ++c4)
          *reinterpret_cast<uint4*>(stage + (c4 * 32 + lane) * 16) =
              make_uint4(o[(4 * c4) >> 5][(4 * c4) & 31], o[(4 * c4) >> 5][(4 * c4 + 1) & 31],
                         o[(4 * c4) >> 5][(4 * c4 + 2) & 31], o[(4 * c4) >> 5][(4 * c4 + 3) & 31]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          const int64_t blk = dq_block_index(a.cu_seqlens_q != nullptr, b, hq, a.heads, (int)si.q_row0, P.dq_blocks) + mblk_of(it);
          float* gdst = a.dq_accum + ((blk * 2 + w) * 4 + (warp & 3)) * (int64_t)(kWarpBytes / 4);
          if (!(P.debug & 1)) bulk_reduce_add_f32(gdst, smem_addr(stage), kWarpBytes);
          bulk_commit_wait_read();
          mbar_arrive(bar_qdo_empty(slot));  // the staging bytes have been read: the slot may be refilled
        }
      }
    }

    if (lane == 0) bulk_wait_all();  // the dQ reductions of this warp have been performed
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
    setmaxnreg_dec<72>();
    if (warp == 8) {
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
        for (int it = 0; it < iters && ok; ++it) {
          const int slot = it & 1, round = it >> 1;
          ok = mbar_wait(bar_qdo_empty(slot), (round & 1) ^ 1, W_B_QDO_EMPTY, abort_flag);
          if (!ok) break;
          const int row = (int)si.q_row0 + mblk_of(it) * kB, hq = head_of(it);
          mbar_expect_tx(bar_qdo_full(slot), 2 * C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c) {
            tma_load_4d(sQ(slot) + c * kChunkBytes, &P.tq, bar_qdo_full(slot), c * 64, row, hq, qb);
            tma_load_4d(sDO(slot) + c * kChunkBytes, &P.tdo, bar_qdo_full(slot), c * 64, row, hq, qb);
          }
        }
      }
    } else if (warp == 10) {
      // -------------------------------------------------------------- LSE / D loader
      bool ok = run;
      for (int it = 0; it < iters && ok; ++it) {
        const int slot = it & 1, round = it >> 1;
        ok = mbar_wait(bar_st_empty(slot), (round & 1) ^ 1, W_B_STATS_EMPTY, abort_flag);
        if (!ok) break;
        const int m0 = mblk_of(it) * kB, hq = head_of(it);
        const float* lse_g = a.softmax_lse + ((int64_t)b * a.heads + hq) * a.lse_seqlen;
        const float* d_g = a.softmax_d + ((int64_t)b * a.heads + hq) * a.d_seqlen;
        float* dst = sStats + slot * 256;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = i * 32 + lane, q = m0 + r;
          const float l = q < si.sq ? lse_g[q] : INFINITY;
          dst[r] = l * kLog2e;  // +inf stays +inf: exp2(x - inf) = 0 for rows without keys / past the end
          dst[128 + r] = q < si.sq ? d_g[q] : 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_st_full(slot));
      }
    } else if (warp == 9) {
      // -------------------------------------------------------------- MMA issuer
      if (lane == 0 && run) {
        constexpr int F = BFmt<T>::kIdesc;
        constexpr uint32_t idesc_st = make_idesc(kB, kB, F, 0, 0);   // S^T, dP^T: K-major x K-major, N = 128 queries
        constexpr uint32_t idesc_dv = make_idesc(kB, DH, F, 0, 1);   // dV, dK: A K-major (or TMEM), B MN-major, N = DH
        constexpr uint32_t idesc_dq = make_idesc(kB, DH, F, 1, 1);   // dQ: A MN-major, B MN-major
        bool ok = mbar_wait(bar_kv, 0, W_B_KV, abort_flag);
        auto issue_st = [&](uint32_t d_col, uint32_t a_tile, uint32_t b_tile, uint32_t bar) {
#pragma unroll
          for (int kk = 0; kk < DH / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
            mma_ss(tmem + d_col, smem_desc_sw128(a_tile + off, 16, 1024), smem_desc_sw128(b_tile + off, 16, 1024), idesc_st,
                   kk > 0);
          }
          tc_commit(bar);
        };
        if (ok) ok = mbar_wait(bar_qdo_full(0), 0, W_B_QDO_FULL, abort_flag);
        if (ok) {
          tc_fence_after();
          issue_st(C::COL_S, sK, sQ(0), bar_s);
          issue_st(C::COL_DP, sV, sDO(0), bar_dp);
        }
        for (int it = 0; it < iters && ok; ++it) {
          const int slot = it & 1;
          ok = mbar_wait(bar_pds, it & 1, W_B_PDS, abort_flag);
          if (!ok) break;
          tc_fence_after();
          // dV += P^T dO
#pragma unroll
          for (int kk = 0; kk < kB / 16; ++kk)
            mma_ts(tmem + C::COL_DV, tmem + C::COL_S + kk * 8, smem_desc_sw128(sDO(slot) + kk * 2048, kChunkBytes, 1024),
                   idesc_dv, (it > 0) || kk > 0);
          // dK += dS^T Q
#pragma unroll
          for (int kk = 0; kk < kB / 16; ++kk) {
            const uint32_t aoff = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
            if (!(P.debug & 16))
            mma_ss(tmem + C::COL_DK, smem_desc_sw128(sDS + aoff, 16, 1024),
                   smem_desc_sw128(sQ(slot) + kk * 2048, kChunkBytes, 1024), idesc_dv, (it > 0) || kk > 0);
          }
          // dQ = dS K  (over the dP^T columns, which the compute warps have consumed)
#pragma unroll
          for (int kk = 0; kk < kB / 16; ++kk)
            if (!(P.debug & 8))
            mma_ss(tmem + C::COL_DP, smem_desc_sw128(sDS + kk * 2048, kChunkBytes, 1024),
                   smem_desc_sw128(sK + kk * 2048, kChunkBytes, 1024), idesc_dq, kk > 0);
          tc_commit(bar_dq_full);
          tc_commit(bar_qdo_empty(slot));
          if (it + 1 < iters) {
            const int ns = (it + 1) & 1;
            ok = mbar_wait(bar_qdo_full(ns), ((it + 1) >> 1) & 1, W_B_QDO_FULL, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_st(C::COL_S, sK, sQ(ns), bar_s);
            // dP^T(it+1) lands on the columns that still hold dQ(it): wait until it has been drained
            ok = mbar_wait(bar_dq_empty, it & 1, W_B_DQ_EMPTY, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_st(C::COL_DP, sV, sDO(ns), bar_dp);
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
  if (warp == 11) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <typename T, int DH>
int launch_bwd_tc(const FaBwdArgs& a, cudaStream_t st) {
  using C = BCfg<DH>;
  BwdTcParams P;
  P.a = a;
  {
    const char* dbg = getenv("FA_B200_DEBUG_BWD");
    P.debug = dbg ? atoi(dbg) : 0;
    P.dq_blocks = dq_blocks_per_unit(a.cu_seqlens_q != nullptr, a.seqlen_q, a.total_q, a.batch);
  }
  const bool varlen = a.cu_seqlens_q != nullptr;
  const int64_t q_rows = varlen ? a.total_q : a.seqlen_q, k_rows = varlen ? a.total_k : a.seqlen_k;
  const int64_t nb = varlen ? 1 : a.batch;
  if (make_tmap_4d(&P.tq, a.q, a.dtype, q_rows, a.heads, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tdo, a.dout, a.dtype, q_rows, a.heads, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tk, a.k, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kB)) return 1;
  if (make_tmap_4d(&P.tv, a.v, a.dtype, k_rows, a.heads_k, nb, a.head_dim, kB)) return 1;
  auto kern = bwd_tc_kernel<T, DH>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) {
      fa_host::set_error("bwd_tc_kernel: cannot reserve %d bytes of shared memory", C::SMEM_BYTES);
      cudaGetLastError();
      return 2;
    }
    attr_set = true;
  }
  dim3 grid((a.seqlen_k + kB - 1) / kB, a.heads_k, a.batch);
  kern<<<grid, 384, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("bwd_tc_kernel");
}

}  // namespace

bool bwd_tc_eligible(const FaBwdArgs& a) {
  if (a.head_dim > 128 || a.p_dropout > 0.f) return false;
  if (a.seqlen_k <= 0 || a.seqlen_q <= 0) return false;
  if (!tma_compatible(a.q) || !tma_compatible(a.k) || !tma_compatible(a.v) || !tma_compatible(a.dout)) return false;
  if (a.head_dim % 8) return false;
  if (a.cu_seqlens_q && (a.total_q <= 0 || a.total_k <= 0)) return false;
  return encode_tiled_fn() != nullptr;
}

int bwd_tc_main(const FaBwdArgs& a, cudaStream_t st) {
  const bool bf = a.dtype == FA_DTYPE_BF16;
  if (a.head_dim <= 64) return bf ? launch_bwd_tc<__nv_bfloat16, 64>(a, st) : launch_bwd_tc<__half, 64>(a, st);
  return bf ? launch_bwd_tc<__nv_bfloat16, 128>(a, st) : launch_bwd_tc<__half, 128>(a, st);
}

int bwd_tc_status(bool clear) {
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
