// Backward attention on tcgen05 tensor cores (head dim <= 128), part 2 of 2: dQ.
//
// One CTA owns 128 query rows of one (batch, query head), keeps Q and dO in shared memory and dQ in
// tensor memory, and walks every 128-key block those rows can see (bwd_tc.cu holds part 1, dK / dV,
// and says why the pass is split).  Same math as the dQ half of compute_dq_dk_dv_1colblock
// (csrc/flash_attn/src/flash_bwd_kernel.h:425-1112):
//   S   = Q K^T           (lanes = queries, columns = keys)             SS MMA  -> TMEM tS
//   dP  = dO V^T                                                         SS MMA  -> TMEM tdP
//   P   = exp2(S*scale*log2e - LSE*log2e)             one thread per query row, stays in registers
//   dS  = P o (dP - D)                                                   -> TMEM (16-bit, buffer j & 1)
//   dQ += dS K            A = dS from TMEM, B = K tile (MN-major)        -> TMEM tdQ
// S and dP are consumed into registers as soon as they are complete, so the tensor pipe computes
// S(j+1) and dP(j+1) while the compute warps are still working on block j; dS has two buffers of
// its own, so dQ(j) never holds up either of them.
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

StatusRef status_ref(bool may_allocate);

namespace {

constexpr int kB = 128;                 // query rows per CTA == keys per block
constexpr int kChunkBytes = 128 * 128;  // [128 rows][64 x 16-bit]
constexpr int kThreads = 384;
constexpr int kWarpProducer = 8, kWarpMma = 9, kWarpTmem = 10, kWarpMmaDq = 11;
constexpr int kRegsCompute = 200, kRegsOther = 72;

enum DqWait { W_Q_ALIGN = 40, W_Q_QDO = 41, W_Q_KV_FULL = 42, W_Q_KV_EMPTY = 43, W_Q_S = 44, W_Q_DP = 45, W_Q_DS = 46,
              W_Q_DONE = 47 };

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
  static constexpr int NBAR = 2 * NSK + 2 * NSV + 8;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 32;
  static constexpr int COL_S = 0, COL_DP = 128, COL_DS = 256, COL_DQ = 384;  // dS: two 64-column buffers
  static constexpr int TMEM_COLS = 512;
};

struct DqTcParams {
  CUtensorMap tq, tk, tv, tdo;
  FaBwdArgs a;
  StatusRef status;
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
  const uint32_t bar_s = bar0 + 8 * kB0, bar_sread = bar0 + 8 * (kB0 + 1), bar_qdo = bar0 + 8 * (kB0 + 2),
                 bar_dp = bar0 + 8 * (kB0 + 3), bar_ds = bar0 + 8 * (kB0 + 4), bar_done = bar0 + 8 * (kB0 + 5),
                 bar_dpread = bar0 + 8 * (kB0 + 6);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_BAR + C::NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + C::NBAR * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (a.heads / a.heads_k);
  const SeqInfo si = seq_info(a.cu_seqlens_q, a.cu_seqlens_k, nullptr, nullptr, a.seqlen_q, a.seqlen_k,
                              a.use_mask_shift, a.mask_shift, b);
  // heavy query blocks (bottom rows of a causal mask see the most keys) are scheduled first
  const int mblk = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int m0 = mblk * kB;
  if (m0 >= si.sq) return;
  int n_lo, n_hi;
  key_block_range(m0, kB, kB, si.sk, si.shift, a.window_left, a.window_right, n_lo, n_hi);
  const int iters = n_hi - n_lo;

  if (threadIdx.x == 0) {
    abort_init(abort_flag, P.status);
    if (s_base & 1023u) abort_raise(abort_flag, W_Q_ALIGN);  // the swizzled tiles need a 1024-byte aligned base
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
    mbar_init(bar_dpread, 8);
    mbar_init(bar_qdo, 1);
    mbar_init(bar_dp, 1);
    mbar_init(bar_ds, 8);
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
    const int w = warp >> 2;                    // key-column half / head-dim half
    const int r = (warp & 3) * 32 + lane;       // query row of this thread within the CTA tile
    const int qrow = m0 + r;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tdP = tmem + lane_off + C::COL_DP + w * 64;
    bool ok = (*abort_flag == 0);  // with iters == 0 the loop is skipped and the epilogue writes zeros
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
    for (int j = 0; j < iters && ok; ++j) {
      const int n0 = (n_lo + j) * kB;
      const uint32_t tS = tmem + lane_off + C::COL_S + w * 64;
      const bool need_mask = (n0 + kB > si.sk) ||
                             (a.window_right >= 0 && n0 + kB - 1 > m0 + si.shift + a.window_right) ||
                             (a.window_left >= 0 && n0 < m0 + kB - 1 + si.shift - a.window_left);
      // ---- P = exp2(S * scale - LSE), 64 key columns per thread, kept in registers
      ok = mbar_wait(bar_s, j & 1, W_Q_S, abort_flag);
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
        if (lane == 0) mbar_arrive(bar_sread);  // S(j) is in registers: S(j+1) may overwrite it
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
      ok = mbar_wait(bar_dp, j & 1, W_Q_DP, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t d0[32], d1[32], pk[32];
        tmem_ld32(tdP, d0);
        tmem_ld32(tdP + 32, d1);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dpread);  // dP(j) is in registers: dP(j+1) may overwrite it
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float x0 = p[c] * (__uint_as_float(c < 32 ? d0[c & 31] : d1[c & 31]) - dsum);
          const float x1 = p[c + 1] * (__uint_as_float(c < 32 ? d0[(c + 1) & 31] : d1[(c + 1) & 31]) - dsum);
          pk[c >> 1] = Pack<T>::two(x0, x1);
        }
        // the buffer held dS(j-2): dQ(j-2), whose commit releases that block's K tile, must have read it
        if (j >= 2) {
          ok = mbar_wait(bar_k_empty((j - 2) % NSK), ((j - 2) / NSK) & 1, W_Q_KV_EMPTY, abort_flag);
          if (!ok) break;
        }
        tmem_st32(tmem + lane_off + C::COL_DS + (j & 1) * 64 + w * 32, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ds);
    }
    // ---- epilogue: dQ * softmax_scale
    if (ok && iters > 0) ok = mbar_wait(bar_done, 0, W_Q_DONE, abort_flag);
    tc_fence_after();
    if (ok && *abort_flag == 0) {  // warp-uniform: the TMEM loads below are warp-wide instructions
      const uint32_t tdQ = tmem + lane_off + C::COL_DQ + w * (DH / 2);
      T* g = reinterpret_cast<T*>(a.dq.ptr) + si.q_batch * a.dq.stride_b + (si.q_row0 + qrow) * a.dq.stride_s +
             (int64_t)hq * a.dq.stride_h;
      const float sc = a.softmax_scale;
#pragma unroll
      for (int c0 = 0; c0 < DH / 2; c0 += 32) {
        uint32_t o[32];
        if (iters > 0) {
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
            *reinterpret_cast<uint4*>(g + col0 + i) = v;
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
        mbar_expect_tx(bar_qdo, 2 * C::TILE_BYTES);
        for (int c = 0; c < C::NCHUNK; ++c) {
          tma_load_4d(sQ + c * kChunkBytes, &P.tq, bar_qdo, c * 64, (int)si.q_row0 + m0, hq, qb);
          tma_load_4d(sDO + c * kChunkBytes, &P.tdo, bar_qdo, c * 64, (int)si.q_row0 + m0, hq, qb);
        }
        bool ok = true;
        for (int j = 0; j < iters && ok; ++j) {
          const int ks = j % NSK, vs = j % NSV;
          const int row = (int)si.k_row0 + (n_lo + j) * kB;
          ok = mbar_wait(bar_k_empty(ks), ((j / NSK) & 1) ^ 1, W_Q_KV_EMPTY, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bar_k_full(ks), C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c) tma_load_4d(sK(ks) + c * kChunkBytes, &P.tk, bar_k_full(ks), c * 64, row, hk, kb);
          ok = mbar_wait(bar_v_empty(vs), ((j / NSV) & 1) ^ 1, W_Q_KV_EMPTY, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bar_v_full(vs), C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c) tma_load_4d(sV(vs) + c * kChunkBytes, &P.tv, bar_v_full(vs), c * 64, row, hk, kb);
        }
      }
    } else if (warp == kWarpMma || warp == kWarpMmaDq) {
      // -------------------------------------------------------------- MMA issuer
      // Each MMA group is issued as soon as its inputs exist and its output columns are free:
      //   S(j+1) once the compute warps hold S(j) in registers, dP(j+1) once they hold dP(j),
      //   dQ(j) once dS(j) is in its buffer.
      if (run) {  // the whole warp runs the loops (see mma_ss_w); one elected lane issues
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
          for (int kk = 0; kk < DH / 16; ++kk) mma_ss_w(tmem + d_col, dsc(a_lo + koff(kk)), dsc(b_lo + koff(kk)), idesc_s, kk > 0);
          tc_commit_w(bar);
        };
        bool ok = mbar_wait_w(bar_qdo, 0, W_Q_QDO, abort_flag);
        if (warp == kWarpMma) {
          // ---- S and dP: block j+1 as soon as the compute warps hold block j's in registers
          for (int j = 0; j < iters && ok; ++j) {
            const int ks = j % NSK, vs = j % NSV;
            if (j > 0) ok = mbar_wait_w(bar_sread, (j - 1) & 1, W_Q_S, abort_flag);
            if (ok) ok = mbar_wait_w(bar_k_full(ks), (j / NSK) & 1, W_Q_KV_FULL, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_s(C::COL_S, oQ, oK + ks * kTile16, bar_s);
            if (j > 0) ok = mbar_wait_w(bar_dpread, (j - 1) & 1, W_Q_DP, abort_flag);
            if (ok) ok = mbar_wait_w(bar_v_full(vs), (j / NSV) & 1, W_Q_KV_FULL, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_s(C::COL_DP, oDO, oV + vs * kTile16, bar_dp);
            tc_commit_w(bar_v_empty(vs));
          }
        } else {
          // ---- dQ += dS K: the two warpgroups' halves of dS are the two 32-column halves of the block's buffer.
          // Its commit releases the K tile, which S(j) of the other issuer read as well: dS(j) was computed from S(j).
          for (int j = 0; j < iters && ok; ++j) {
            const int ks = j % NSK;
            ok = mbar_wait_w(bar_ds, j & 1, W_Q_DS, abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kB / 16; ++kk)
              mma_ts_w(tmem + C::COL_DQ, tmem + C::COL_DS + (j & 1) * 64 + kk * 8, dsc(oK + ks * kTile16 + moff(kk)), idesc_dq,
                     (j > 0) || kk > 0);
            tc_commit_w(bar_k_empty(ks));
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
  P.status = status_ref(true);
  static fa_host::DeviceOnce once;
  if (int rc = fa_host::raise_smem_limit(once, reinterpret_cast<const void*>(kern), C::SMEM_BYTES, "bwd_dq_tc_kernel")) return rc;
  dim3 grid((a.seqlen_q + kB - 1) / kB, a.heads, a.batch);
  kern<<<grid, kThreads, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("bwd_dq_tc_kernel");
}

}  // namespace

int bwd_dq_tc_main(const FaBwdArgs& a, cudaStream_t st) {
  const bool bf = a.dtype == FA_DTYPE_BF16;
  if (a.head_dim <= 64) return bf ? launch_bwd_dq_tc<__nv_bfloat16, 64>(a, st) : launch_bwd_dq_tc<__half, 64>(a, st);
  return bf ? launch_bwd_dq_tc<__nv_bfloat16, 128>(a, st) : launch_bwd_dq_tc<__half, 128>(a, st);
}

}  // namespace fa
