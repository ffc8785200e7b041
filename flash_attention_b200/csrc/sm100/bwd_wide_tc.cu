// Backward attention on tcgen05 tensor cores for head dims 129..256: three passes of one kernel.
//
// With 256 head-dim columns neither the accumulators (dK and dV alone would fill all 512 columns of
// tensor memory) nor the tiles (four 128 x 256 tiles are 256 KiB) of the 128-wide kernels
// (bwd_tc.cu, bwd_dq_tc.cu) fit, so each output gets a pass of its own.  A CTA keeps 128 rows of the
// "stationary" side in shared memory, its 128 x 256 fp32 result in tensor memory, and streams the
// other side past them in blocks of 64 rows.  Same math as compute_dq_dk_dv_1colblock
// (csrc/flash_attn/src/flash_bwd_kernel.h:425-1112):
//   pass dV: stationary K;      stream Q, dO;  X1 = K Q^T (= S^T);                 W = P^T;   dV += W dO
//   pass dK: stationary K, V;   stream Q, dO;  X1 = K Q^T, X2 = V dO^T (= dP^T);   W = dS^T;  dK += W Q
//   pass dQ: stationary Q, dO;  stream K, V;   X1 = Q K^T, X2 = dO V^T;            W = dS;    dQ += W K
// with P = exp2(S*scale*log2e - LSE*log2e) and dS = P o (dP - D).  X1 / X2 (128 lanes x 64 fp32
// columns) are consumed into registers as soon as they complete; W goes back to tensor memory as
// the 16-bit A operand of the last product (two buffers), whose B operand is the streamed tile read
// MN-major.  No atomics: every output element is written by exactly one CTA.
//
// Warps: 0-7 compute (warpgroup w handles streamed columns [32w, 32w+32) of a block; in the
// epilogue, head-dim columns [128w, 128w+128)), 8 = TMA producer, 9 and 11 = MMA issuers, 10 = TMEM owner.
#include <cstdlib>

#include "../fa_common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace fa {

using namespace ptx;

StatusRef status_ref(bool may_allocate);

namespace {

constexpr int kR = 128;                  // stationary rows per CTA
constexpr int kN = 64;                   // streamed rows per block
constexpr int kDH = 256;                 // padded head dim
constexpr int kChunkA = kR * 128;        // [128 rows][64 x 16-bit]
constexpr int kChunkB = kN * 128;        // [64 rows][64 x 16-bit]
constexpr int kTileA = 4 * kChunkA, kTileB = 4 * kChunkB;
constexpr int kThreads = 384;
constexpr int kWarpProducer = 8, kWarpMma = 9, kWarpTmem = 10, kWarpMmaX1 = 11;
constexpr int kRegsCompute = 200, kRegsOther = 72;

enum Pass { PASS_DV = 0, PASS_DK = 1, PASS_DQ = 2 };

enum WWait { W_W_ALIGN = 60, W_W_A = 61, W_W_B_FULL = 62, W_W_B_EMPTY = 63, W_W_X1 = 64, W_W_X2 = 65, W_W_W = 66,
             W_W_DONE = 67, W_W_READ = 68 };

template <int PASS>
struct WCfg {
  static constexpr int NA = PASS == PASS_DV ? 1 : 2;
  // passes dK / dQ: B1 is held from X1(j) (issued a block early) to the last product of block j, B2 only by X2(j);
  // pass dV: B1 (Q) only by X1(j), B2 (dO) from its arrival to the last product of block j
  static constexpr int NS1 = 2;
  static constexpr int NS2 = PASS == PASS_DV ? 3 : 1;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B1 = NA * kTileA;
  static constexpr int OFF_B2 = OFF_B1 + NS1 * kTileB;
  static constexpr int OFF_STATS = OFF_B2 + NS2 * kTileB;  // per compute warp: 32 LSE + 32 D of the streamed columns
  static constexpr int STATS_BYTES = PASS == PASS_DQ ? 0 : 8 * 64 * 4;
  static constexpr int OFF_BAR = OFF_STATS + STATS_BYTES;
  static constexpr int NBAR = 2 * NS1 + 2 * NS2 + 8;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 32;
  static constexpr int COL_X1 = 0, COL_X2 = 64, COL_W = 128, COL_OUT = 256;  // W: two 32-column buffers
  static constexpr int TMEM_COLS = 512;
  static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA");
};

struct WParams {
  CUtensorMap ta1, ta2, tb1, tb2;  // stationary tiles (128-row boxes), streamed tiles (64-row boxes)
  FaBwdArgs a;
  StatusRef status;
};

template <typename T>
struct WFmt;
template <>
struct WFmt<__half> {
  static constexpr int kIdesc = 0;
};
template <>
struct WFmt<__nv_bfloat16> {
  static constexpr int kIdesc = 1;
};

// Position in the stream of passes dV / dK: query blocks [m_lo, m_hi) of every query head of the group
struct Walk {
  int mb, hq, m_lo, m_hi;
  __device__ __forceinline__ void next() {
    if (++mb == m_hi) {
      mb = m_lo;
      ++hq;
    }
  }
};

template <typename T, int PASS>
__global__ void __launch_bounds__(kThreads, 1) bwd_wide_tc_kernel(const __grid_constant__ WParams P) {
  using C = WCfg<PASS>;
  constexpr int NS1 = C::NS1, NS2 = C::NS2;
  constexpr bool kRowsAreQueries = PASS == PASS_DQ;
  const FaBwdArgs& a = P.a;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t s_base = smem_addr(smem);
  auto sB1 = [&](int st) { return s_base + C::OFF_B1 + st * kTileB; };
  auto sB2 = [&](int st) { return s_base + C::OFF_B2 + st * kTileB; };
  const uint32_t bar0 = s_base + C::OFF_BAR;
  auto bar_b1_full = [&](int st) { return bar0 + 8 * st; };
  auto bar_b1_empty = [&](int st) { return bar0 + 8 * (NS1 + st); };
  auto bar_b2_full = [&](int st) { return bar0 + 8 * (2 * NS1 + st); };
  auto bar_b2_empty = [&](int st) { return bar0 + 8 * (2 * NS1 + NS2 + st); };
  constexpr int kB0 = 2 * NS1 + 2 * NS2;
  const uint32_t bar_x1 = bar0 + 8 * kB0, bar_x1read = bar0 + 8 * (kB0 + 1), bar_a = bar0 + 8 * (kB0 + 2),
                 bar_x2 = bar0 + 8 * (kB0 + 3), bar_x2read = bar0 + 8 * (kB0 + 4), bar_w = bar0 + 8 * (kB0 + 5),
                 bar_done = bar0 + 8 * (kB0 + 6);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_BAR + C::NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + C::NBAR * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int group = a.heads / a.heads_k;
  const SeqInfo si = seq_info(a.cu_seqlens_q, a.cu_seqlens_k, nullptr, nullptr, a.seqlen_q, a.seqlen_k,
                              a.use_mask_shift, a.mask_shift, b);
  // r0: first stationary row; [c_lo_blk, c_hi_blk): streamed 64-row blocks these rows can see
  int r0, blk_lo, blk_hi, iters, hq_fixed, hk;
  if (kRowsAreQueries) {
    hq_fixed = blockIdx.y;
    hk = hq_fixed / group;
    r0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kR;  // heavy query blocks of a causal mask first
    if (r0 >= si.sq) return;
    key_block_range(r0, kR, kN, si.sk, si.shift, a.window_left, a.window_right, blk_lo, blk_hi);
    iters = blk_hi - blk_lo;
  } else {
    hk = blockIdx.y;
    hq_fixed = hk * group;
    r0 = blockIdx.x * kR;
    if (r0 >= si.sk) return;
    query_block_range(r0, kR, kN, si.sq, si.shift, a.window_left, a.window_right, blk_lo, blk_hi);
    iters = (blk_hi - blk_lo) * group;
  }

  if (threadIdx.x == 0) {
    abort_init(abort_flag, P.status);
    if (s_base & 1023u) abort_raise(abort_flag, W_W_ALIGN);  // the swizzled tiles need a 1024-byte aligned base
    for (int s = 0; s < NS1; ++s) {
      mbar_init(bar_b1_full(s), 1);
      mbar_init(bar_b1_empty(s), 1);
    }
    for (int s = 0; s < NS2; ++s) {
      mbar_init(bar_b2_full(s), 1);
      mbar_init(bar_b2_empty(s), 1);
    }
    mbar_init(bar_x1, 1);
    mbar_init(bar_x1read, 8);
    mbar_init(bar_a, 1);
    mbar_init(bar_x2, 1);
    mbar_init(bar_x2read, 8);
    mbar_init(bar_w, 8);
    mbar_init(bar_done, 1);
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
  const bool run = (*abort_flag == 0) && iters > 0;
  const float scale_log2 = a.softmax_scale * kLog2e;

  if (warp < 8) {
    // ---------------------------------------------------------------- compute warpgroups
    setmaxnreg_inc<kRegsCompute>();
    const int w = warp >> 2;               // streamed-column half / head-dim half
    const int r = (warp & 3) * 32 + lane;  // stationary row of this thread within the CTA tile
    const int row = r0 + r;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tX1 = tmem + lane_off + C::COL_X1 + w * 32, tX2 = tmem + lane_off + C::COL_X2 + w * 32;
    bool ok = (*abort_flag == 0);  // with iters == 0 the loop is skipped and the epilogue writes zeros
    const float* lse_base = a.softmax_lse + (int64_t)b * a.heads * a.lse_seqlen;
    const float* d_base = a.softmax_d + (int64_t)b * a.heads * a.d_seqlen;
    // pass dQ: statistics of this thread's own query row; +inf LSE (rows past the end or without keys) gives P = 0
    float lse2 = INFINITY, dsum = 0.f;
    int k_lo = 0, k_hi = si.sk - 1;  // keys this query row can see
    if (kRowsAreQueries) {
      if (row < si.sq) {
        lse2 = lse_base[(int64_t)hq_fixed * a.lse_seqlen + row] * kLog2e;
        dsum = d_base[(int64_t)hq_fixed * a.d_seqlen + row];
      }
      if (a.window_right >= 0) k_hi = min(k_hi, row + si.shift + a.window_right);
      if (a.window_left >= 0) k_lo = max(k_lo, row + si.shift - a.window_left);
    }
    // passes dV / dK: statistics of the 32 streamed query columns of this warp, one per lane, staged through
    // this warp's own 256 bytes of shared memory; the next block's values are fetched a block ahead
    float* st = reinterpret_cast<float*>(smem + C::OFF_STATS) + warp * 64;
    Walk wk{blk_lo, hq_fixed, blk_lo, blk_hi};
    float nl = INFINITY, nd = 0.f;
    auto load_stats = [&](const Walk& k) {
      const int m = k.mb * kN + w * 32 + lane;
      nl = INFINITY;
      nd = 0.f;
      if (m < si.sq) {
        nl = lse_base[(int64_t)k.hq * a.lse_seqlen + m];  // scaled when it is staged: no use of the value here
        if (PASS != PASS_DV) nd = d_base[(int64_t)k.hq * a.d_seqlen + m];
      }
    };
    if (!kRowsAreQueries && iters > 0) load_stats(wk);

    for (int it = 0; it < iters && ok; ++it) {
      int c0;  // first streamed row of this block
      if (kRowsAreQueries) {
        c0 = (blk_lo + it) * kN;
      } else {
        c0 = wk.mb * kN;
        __syncwarp();
        st[lane] = nl * kLog2e;
        st[32 + lane] = nd;
        __syncwarp();
        wk.next();
        if (it + 1 < iters) load_stats(wk);
      }
      // visible streamed columns of this thread's row, relative to the warpgroup's first column: [c_lo, c_hi]
      int c_lo, c_hi;
      bool need_mask;
      if (kRowsAreQueries) {
        c_lo = k_lo - c0 - w * 32;
        c_hi = k_hi - c0 - w * 32;
        need_mask = (c0 + kN > si.sk) || (a.window_right >= 0 && c0 + kN - 1 > r0 + si.shift + a.window_right) ||
                    (a.window_left >= 0 && c0 < r0 + kR - 1 + si.shift - a.window_left);
      } else {
        c_lo = 0;
        c_hi = min(kN, si.sq - c0) - 1;
        if (a.window_right >= 0) c_lo = max(c_lo, row - si.shift - a.window_right - c0);
        if (a.window_left >= 0) c_hi = min(c_hi, row - si.shift + a.window_left - c0);
        if (row >= si.sk) c_hi = -1;
        c_lo -= w * 32;
        c_hi -= w * 32;
        need_mask = (r0 + kR > si.sk) || (c0 + kN > si.sq) ||
                    (a.window_right >= 0 && r0 + kR - 1 > c0 + si.shift + a.window_right) ||
                    (a.window_left >= 0 && r0 < c0 + kN - 1 + si.shift - a.window_left);
      }
      // ---- X2 completes first (see the MMA issuer): it is taken into registers right away so that X2(it+1) can go
      uint32_t d[32];
      if (PASS != PASS_DV) {
        ok = mbar_wait(bar_x2, it & 1, W_W_X2, abort_flag);
        if (!ok) break;
        tc_fence_after();
        tmem_ld32(tX2, d);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_x2read);  // X2(it) is in registers: X2(it+1) may overwrite it
      }
      // ---- P = exp2(X1 * scale - LSE), 32 streamed columns per thread, kept in registers
      ok = mbar_wait(bar_x1, it & 1, W_W_X1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      float p[32];
      {
        uint32_t s[32];
        tmem_ld32(tX1, s);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_x1read);  // X1(it) is in registers: X1(it+1) may overwrite it
        if (kRowsAreQueries) {
#pragma unroll
          for (int c = 0; c < 32; ++c) p[c] = ex2(fmaf(__uint_as_float(s[c]), scale_log2, -lse2));
        } else {
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) {
            const float4 l4 = reinterpret_cast<const float4*>(st)[c4];
            p[c4 * 4 + 0] = ex2(fmaf(__uint_as_float(s[c4 * 4 + 0]), scale_log2, -l4.x));
            p[c4 * 4 + 1] = ex2(fmaf(__uint_as_float(s[c4 * 4 + 1]), scale_log2, -l4.y));
            p[c4 * 4 + 2] = ex2(fmaf(__uint_as_float(s[c4 * 4 + 2]), scale_log2, -l4.z));
            p[c4 * 4 + 3] = ex2(fmaf(__uint_as_float(s[c4 * 4 + 3]), scale_log2, -l4.w));
          }
        }
      }
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 32; ++c) p[c] = (c >= c_lo && c <= c_hi) ? p[c] : 0.f;
      }
      uint32_t pk[16];
      if (PASS == PASS_DV) {
#pragma unroll
        for (int c = 0; c < 32; c += 2) pk[c >> 1] = Pack<T>::two(p[c], p[c + 1]);
      } else {
        // ---- dS = P o (X2 - D)
        if (kRowsAreQueries) {
#pragma unroll
          for (int c = 0; c < 32; c += 2)
            pk[c >> 1] = Pack<T>::two(p[c] * (__uint_as_float(d[c]) - dsum), p[c + 1] * (__uint_as_float(d[c + 1]) - dsum));
        } else {
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) {
            const float4 d4 = reinterpret_cast<const float4*>(st + 32)[c4];
            pk[c4 * 2] = Pack<T>::two(p[c4 * 4] * (__uint_as_float(d[c4 * 4]) - d4.x),
                                      p[c4 * 4 + 1] * (__uint_as_float(d[c4 * 4 + 1]) - d4.y));
            pk[c4 * 2 + 1] = Pack<T>::two(p[c4 * 4 + 2] * (__uint_as_float(d[c4 * 4 + 2]) - d4.z),
                                          p[c4 * 4 + 3] * (__uint_as_float(d[c4 * 4 + 3]) - d4.w));
          }
        }
      }
      // the buffer held W(it-2): the product that read it, whose commit releases that block's tile, must be complete
      if (it >= 2) {
        if (PASS == PASS_DV)
          ok = mbar_wait(bar_b2_empty((it - 2) % NS2), ((it - 2) / NS2) & 1, W_W_B_EMPTY, abort_flag);
        else
          ok = mbar_wait(bar_b1_empty((it - 2) % NS1), ((it - 2) / NS1) & 1, W_W_B_EMPTY, abort_flag);
        if (!ok) break;
      }
      tmem_st16(tmem + lane_off + C::COL_W + (it & 1) * 32 + w * 16, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_w);
    }
    // ---- epilogue: the accumulator (times softmax_scale for dQ and dK) goes to its tensor
    if (ok && iters > 0) ok = mbar_wait(bar_done, 0, W_W_DONE, abort_flag);
    tc_fence_after();
    ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);  // the TMEM loads below are warp-wide instructions
    if (ok) {
      const uint32_t tO = tmem + lane_off + C::COL_OUT + w * 128;
      const bool valid = row < (kRowsAreQueries ? si.sq : si.sk);
      const float sc = PASS == PASS_DV ? 1.f : a.softmax_scale;
      const FaTensor& tt = PASS == PASS_DQ ? a.dq : (PASS == PASS_DK ? a.dk : a.dv);
      const int64_t tb = kRowsAreQueries ? si.q_batch : si.k_batch, trow = (kRowsAreQueries ? si.q_row0 : si.k_row0) + row;
      const int th = kRowsAreQueries ? hq_fixed : hk;
      const bool to_accum = !kRowsAreQueries && a.accumulate_dkv;
      T* g = to_accum ? nullptr : reinterpret_cast<T*>(tt.ptr) + tb * tt.stride_b + trow * tt.stride_s + (int64_t)th * tt.stride_h;
      float* acc = to_accum ? (PASS == PASS_DK ? a.dk_accum : a.dv_accum) +
                                  (((int64_t)si.k_batch * a.seqlen_k + si.k_row0 + row) * a.heads_k + hk) * a.head_dim
                            : nullptr;
#pragma unroll
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t o[32];
        if (iters > 0) {
          tmem_ld32(tO + c0, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (!valid) continue;
        const int col0 = w * 128 + c0;
        if (to_accum) {
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
  } else {
    setmaxnreg_dec<kRegsOther>();
    if (warp == kWarpProducer) {
      // -------------------------------------------------------------- TMA producer
      if (lane == 0 && run) {
        prefetch_tensormap(&P.ta1);
        if (C::NA == 2) prefetch_tensormap(&P.ta2);
        prefetch_tensormap(&P.tb1);
        prefetch_tensormap(&P.tb2);
        const int kb = (int)si.k_batch, qb = (int)si.q_batch;
        const int arow = (int)(kRowsAreQueries ? si.q_row0 : si.k_row0) + r0;
        const int ahead = kRowsAreQueries ? hq_fixed : hk, ab = kRowsAreQueries ? qb : kb;
        mbar_expect_tx(bar_a, C::NA * kTileA);
        for (int c = 0; c < 4; ++c) {
          tma_load_4d(s_base + C::OFF_A + c * kChunkA, &P.ta1, bar_a, c * 64, arow, ahead, ab);
          if (C::NA == 2) tma_load_4d(s_base + C::OFF_A + kTileA + c * kChunkA, &P.ta2, bar_a, c * 64, arow, ahead, ab);
        }
        Walk wk{blk_lo, hq_fixed, blk_lo, blk_hi};
        bool ok = true;
        for (int it = 0; it < iters && ok; ++it) {
          const int s1 = it % NS1, s2 = it % NS2;
          int brow, bhead, bb;
          if (kRowsAreQueries) {
            brow = (int)si.k_row0 + (blk_lo + it) * kN;
            bhead = hk;
            bb = kb;
          } else {
            brow = (int)si.q_row0 + wk.mb * kN;
            bhead = wk.hq;
            bb = qb;
            wk.next();
          }
          // in the order the MMA issuer needs them: pass dV X1 (B1) first, passes dK / dQ X2 (B2) first
          for (int step = 0; step < 2 && ok; ++step) {
            const bool first = (step == 0) == (PASS == PASS_DV);
            if (first) {
              ok = mbar_wait(bar_b1_empty(s1), ((it / NS1) & 1) ^ 1, W_W_B_EMPTY, abort_flag);
              if (!ok) break;
              mbar_expect_tx(bar_b1_full(s1), kTileB);
              for (int c = 0; c < 4; ++c) tma_load_4d(sB1(s1) + c * kChunkB, &P.tb1, bar_b1_full(s1), c * 64, brow, bhead, bb);
            } else {
              ok = mbar_wait(bar_b2_empty(s2), ((it / NS2) & 1) ^ 1, W_W_B_EMPTY, abort_flag);
              if (!ok) break;
              mbar_expect_tx(bar_b2_full(s2), kTileB);
              for (int c = 0; c < 4; ++c) tma_load_4d(sB2(s2) + c * kChunkB, &P.tb2, bar_b2_full(s2), c * 64, brow, bhead, bb);
            }
          }
        }
      }
    } else if (warp == kWarpMma || warp == kWarpMmaX1) {
      // -------------------------------------------------------------- MMA issuer
      // Two issuing threads: warp 11 issues the X1 products, warp 9 the X2 products and the last product of every
      // block.  MMAs of different threads are not ordered among themselves, and need not be: each group waits on the
      // barriers of what it reads and overwrites.  One thread alone is blocked while the pipe works through its
      // MMAs (an N = 64 MMA costs it 56 cycles, two threads together 48 per MMA) and cannot look at the next
      // group's barriers meanwhile.
      //   X1(j+1): once the compute warps hold X1(j) in registers and the tile has landed
      //   X2(j+1): once they hold X2(j) and its tile has landed
      //   last product of block j: once W(j) is in its buffer; its commit releases the tile X1(j) read as well
      //   (X1(j) is complete by then: W(j) was computed from it)
      if (run) {  // the whole warp runs the loops (see mma_ss_w); one elected lane issues
        constexpr int F = WFmt<T>::kIdesc;
        constexpr uint32_t idesc_x = make_idesc(kR, kN, F, 0, 0);    // X1, X2: K-major x K-major, N = 64 streamed rows
        constexpr uint32_t idesc_o = make_idesc(kR, kDH, F, 0, 1);   // last product: A in TMEM, B MN-major, N = 256
        // One descriptor is built (first stationary tile, K-major); every other operand differs from it only
        // in the low word: the address field (+ byte offset >> 4) and, for MN-major reads, the LBO field.
        const uint64_t d_base = smem_desc_sw128(s_base + C::OFF_A, 16, 1024);
        const uint32_t d_lo = (uint32_t)d_base, d_hi = (uint32_t)(d_base >> 32);
        auto dsc = [&](uint32_t lo_add) { return ((uint64_t)d_hi << 32) | (uint64_t)(d_lo + lo_add); };
        constexpr uint32_t kMn = (uint32_t)((kChunkB - 16) >> 4) << 16;  // K-major -> MN-major (LBO = chunk stride)
        constexpr uint32_t oA1 = 0, oA2 = kTileA >> 4, oB1 = (C::OFF_B1 - C::OFF_A) >> 4, oB2 = (C::OFF_B2 - C::OFF_A) >> 4,
                           kTileB16 = kTileB >> 4;
        auto koff_a = [](int kk) { return (uint32_t)(((kk >> 2) * kChunkA + (kk & 3) * 32) >> 4); };
        auto koff_b = [](int kk) { return (uint32_t)(((kk >> 2) * kChunkB + (kk & 3) * 32) >> 4); };
        auto moff = [](int kk) { return (uint32_t)((kk * 2048) >> 4) + kMn; };  // MN-major k-step: 16 rows of 128 bytes
        auto issue_x = [&](uint32_t d_col, uint32_t a_lo, uint32_t b_lo) {
#pragma unroll
          for (int kk = 0; kk < kDH / 16; ++kk)
            mma_ss_w(tmem + d_col, dsc(a_lo + koff_a(kk)), dsc(b_lo + koff_b(kk)), idesc_x, kk > 0);
        };
        auto issue_out = [&](int j, uint32_t b_lo) {
          // the two warpgroups' halves of W are the two 16-column halves of this block's buffer
#pragma unroll
          for (int kk = 0; kk < kN / 16; ++kk)
            mma_ts_w(tmem + C::COL_OUT, tmem + C::COL_W + (j & 1) * 32 + kk * 8, dsc(b_lo + moff(kk)), idesc_o, (j > 0) || kk > 0);
        };
        bool ok = mbar_wait_w(bar_a, 0, W_W_A, abort_flag);
        if (warp == kWarpMmaX1) {
          // ---- X1 products
          for (int j = 0; j < iters && ok; ++j) {
            const int s1 = j % NS1;
            if (j > 0) ok = mbar_wait_w(bar_x1read, (j - 1) & 1, W_W_READ, abort_flag);
            if (ok) ok = mbar_wait_w(bar_b1_full(s1), (j / NS1) & 1, W_W_B_FULL, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_x(C::COL_X1, oA1, oB1 + s1 * kTileB16);
            tc_commit_w(bar_x1);
            if (PASS == PASS_DV) tc_commit_w(bar_b1_empty(s1));
          }
        } else {
          // ---- X2 products and the last product of every block
          if (PASS != PASS_DV) {
            if (ok) ok = mbar_wait_w(bar_b2_full(0), 0, W_W_B_FULL, abort_flag);
            if (ok) {
              tc_fence_after();
              issue_x(C::COL_X2, oA2, oB2);
              tc_commit_w(bar_x2);
              tc_commit_w(bar_b2_empty(0));
            }
          }
          for (int j = 0; j < iters && ok; ++j) {
            if (PASS != PASS_DV && j + 1 < iters) {
              const int n2 = (j + 1) % NS2;
              ok = mbar_wait_w(bar_x2read, j & 1, W_W_READ, abort_flag);
              if (ok) ok = mbar_wait_w(bar_b2_full(n2), ((j + 1) / NS2) & 1, W_W_B_FULL, abort_flag);
              if (!ok) break;
              tc_fence_after();
              issue_x(C::COL_X2, oA2, oB2 + n2 * kTileB16);
              tc_commit_w(bar_x2);
              tc_commit_w(bar_b2_empty(n2));
            }
            ok = mbar_wait_w(bar_w, j & 1, W_W_W, abort_flag);
            if (ok && PASS == PASS_DV) ok = mbar_wait_w(bar_b2_full(j % NS2), (j / NS2) & 1, W_W_B_FULL, abort_flag);
            if (!ok) break;
            tc_fence_after();
            if (PASS == PASS_DV) {
              issue_out(j, oB2 + (j % NS2) * kTileB16);
              tc_commit_w(bar_b2_empty(j % NS2));
            } else {
              issue_out(j, oB1 + (j % NS1) * kTileB16);
              tc_commit_w(bar_b1_empty(j % NS1));
            }
          }
          if (ok) tc_commit_w(bar_done);
        }
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {  // copies may still be in flight: give them time before the shared memory goes away
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == kWarpTmem) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <typename T, int PASS>
int launch_wide(const FaBwdArgs& a, cudaStream_t st) {
  using C = WCfg<PASS>;
  WParams P;
  P.a = a;
  const bool varlen = a.cu_seqlens_q != nullptr;
  const int64_t q_rows = varlen ? a.total_q : a.seqlen_q, k_rows = varlen ? a.total_k : a.seqlen_k;
  const int64_t nb = varlen ? 1 : a.batch;
  const int bq = PASS == PASS_DQ ? kR : kN, bk = PASS == PASS_DQ ? kN : kR;
  CUtensorMap tq, tdo, tk, tv;
  if (make_tmap_4d(&tq, a.q, a.dtype, q_rows, a.heads, nb, a.head_dim, bq)) return 1;
  if (make_tmap_4d(&tdo, a.dout, a.dtype, q_rows, a.heads, nb, a.head_dim, bq)) return 1;
  if (make_tmap_4d(&tk, a.k, a.dtype, k_rows, a.heads_k, nb, a.head_dim, bk)) return 1;
  if (make_tmap_4d(&tv, a.v, a.dtype, k_rows, a.heads_k, nb, a.head_dim, bk)) return 1;
  if (PASS == PASS_DQ) {
    P.ta1 = tq, P.ta2 = tdo, P.tb1 = tk, P.tb2 = tv;
  } else {
    P.ta1 = tk, P.ta2 = tv, P.tb1 = tq, P.tb2 = tdo;
  }
  auto kern = bwd_wide_tc_kernel<T, PASS>;
  P.status = status_ref(true);
  static fa_host::DeviceOnce once;
  if (int rc = fa_host::raise_smem_limit(once, reinterpret_cast<const void*>(kern), C::SMEM_BYTES, "bwd_wide_tc_kernel")) return rc;
  dim3 grid(((PASS == PASS_DQ ? a.seqlen_q : a.seqlen_k) + kR - 1) / kR, PASS == PASS_DQ ? a.heads : a.heads_k, a.batch);
  kern<<<grid, kThreads, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("bwd_wide_tc_kernel");
}

template <typename T>
int run_wide(const FaBwdArgs& a, int parts, cudaStream_t st) {
  int rc = 0;
  if (parts & 2) {
    rc = launch_wide<T, PASS_DV>(a, st);
    if (!rc) rc = launch_wide<T, PASS_DK>(a, st);
  }
  if (!rc && (parts & 1)) rc = launch_wide<T, PASS_DQ>(a, st);
  return rc;
}

}  // namespace

// dV, dK (parts & 2) and dQ (parts & 1) of a backward pass with 128 < head_dim <= 256 (softmax_d must hold
// rowsum(dO o O)).
int bwd_wide_tc_main(const FaBwdArgs& a, int parts, cudaStream_t st) {
  return a.dtype == FA_DTYPE_BF16 ? run_wide<__nv_bfloat16>(a, parts, st) : run_wide<__half>(a, parts, st);
}

}  // namespace fa
