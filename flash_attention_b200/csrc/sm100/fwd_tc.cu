// Forward attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head dim <= 256.
//
// One CTA owns 256 query rows of one (batch, head) [and, with split-KV, one range of key blocks]: two
// 128-row tiles that take turns on the tensor pipe (head dims above 128: one tile, because O alone
// fills 256 TMEM columns; warps 4-7 idle).  CTAs are launched heaviest first (bottom rows of a causal
// mask see the most keys).
// Warp roles (384 threads):
//   warps 0-3   softmax of tile 0  (one thread per query row; tcgen05.ld 32x32b gives a thread its row)
//   warps 4-7   softmax of tile 1
//   warp  8     TMA producer: Q tiles once, then K(j), V(j), K(j+1), ... through a ring of slots
//   warp  9     MMA issuer: the warp stays converged, one elected lane issues every tcgen05.mma
//   warp  10    owns the TMEM allocation
// TMEM columns (fp32): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).  P (16-bit) is
// written over the first 64 columns of its S and fed to the PV MMA as the TMEM A operand.
// MMA order  S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) | ...  so that while one tile is in its
// softmax the other tile's two MMAs keep the tensor pipe busy; the single in-order issuer is also what
// keeps the two tiles' softmax phases apart (issuers per tile drift into phase and then share the
// exponential unit).  P is handed over in two halves of 64 keys, each followed by its four k-steps
// of PV.
// Softmax works in the exp2 domain with a lazily updated reference maximum: O and the row sum are
// only rescaled when the running maximum has grown by more than 2^8, which keeps the (expensive)
// TMEM round trip of O off the common path; the final O/l and LSE do not depend on that choice.
// Blocks that the mask touches run a second instance of the block code that classifies each 32-column
// chunk for the warp: a chunk that every row sees is left alone, one that no row sees is skipped (no
// exponentials), only the chunks on the mask boundary are tested element by element.  (One instance for
// all blocks, or a masking pre-pass in front of the straight-line code, both measured slower.)
//
// Split-KV (num_splits > 1): the CTA takes one range of key blocks; its normalised partial O and its
// LSE go to the fp32 workspaces and combine.cu merges them (flash_api.cpp:373-389,
// flash_fwd_launch_template.h:70-138).
//
// A persistent form (one CTA per SM drawing items from a counter, the next item's first S behind the
// current item's last PV, a separate epilogue warpgroup or the softmax warps draining O) was built and
// measured: 0.47 ms against 0.40 ms on 16 x 2048 x 16 x 128 causal, 1163 against 1215 TFLOP/s on
// 2 x 8192 full.  The issuing warp pays hundreds of cycles for every barrier test next to warps that
// are busy with exponentials, and the extra item bookkeeping in that warp cost more than the
// overlapped prologue and epilogue gave back.
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

enum WaitCode { W_QFULL = 11, W_KVFULL = 12, W_KVEMPTY = 13, W_SFULL = 14, W_PFULL = 15, W_OFULL = 16 };

template <int DH>
struct Cfg {
  static constexpr int NCHUNK = DH / 64;
  static constexpr int TILE_BYTES = NCHUNK * kChunkBytes;
  // Head dims up to 128: two 128-row query tiles per CTA ping-pong on the tensor pipe.  Up to 256: O alone
  // needs 256 TMEM columns and a tile is 64 KiB, so one query tile per CTA and a 2-slot (K, V) ring.
  static constexpr int NT = DH > 128 ? 1 : 2;
  static constexpr int STAGES = DH > 128 ? 2 : (DH == 128 ? 4 : 8);
  static constexpr int SMEM_TILES = (NT + STAGES) * TILE_BYTES;
  static constexpr int NBAR = 2 + 2 * STAGES + 8;
  static constexpr int SMEM_BYTES = SMEM_TILES + NBAR * 8 + 32 + 1024;  // + barriers, tmem ptr / abort block, align slack
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S0 = 0, COL_S1 = 128, COL_O0 = 256, COL_O1 = 256 + DH;
};

struct FwdTcParams {
  CUtensorMap tq, tk, tv;
  FaFwdArgs a;
  StatusRef status;
  int32_t num_splits, blocks_per_split;  // split-KV: key blocks [split * blocks_per_split, +blocks_per_split)
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

template <typename T, int DH>
__global__ void __launch_bounds__(384, 1) fwd_tc_kernel(const __grid_constant__ FwdTcParams P) {
  using C = Cfg<DH>;
  const FaFwdArgs& a = P.a;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_addr(smem);
  const uint32_t sQ = s_base;                          // NT tiles
  const uint32_t sKV = s_base + C::NT * C::TILE_BYTES;  // STAGES slots
  const uint32_t bar0 = s_base + C::SMEM_TILES;
  auto bar_qfull = [&](int t) { return bar0 + 8 * t; };
  auto bar_full = [&](int s) { return bar0 + 8 * (2 + s); };
  auto bar_empty = [&](int s) { return bar0 + 8 * (2 + C::STAGES + s); };
  auto bar_sfull = [&](int t) { return bar0 + 8 * (2 + 2 * C::STAGES + t); };
  auto bar_pfull = [&](int t) { return bar0 + 8 * (2 + 2 * C::STAGES + 2 + t); };
  auto bar_ofull = [&](int t) { return bar0 + 8 * (2 + 2 * C::STAGES + 4 + t); };
  auto bar_pfull_b = [&](int t) { return bar0 + 8 * (2 + 2 * C::STAGES + 6 + t); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + C::SMEM_TILES + C::NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::SMEM_TILES + C::NBAR * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 8 * 32) {  // the TMA unit fetches the three descriptors while the CTA sets itself up
    prefetch_tensormap(&P.tq);
    prefetch_tensormap(&P.tk);
    prefetch_tensormap(&P.tv);
  }
  const int b = blockIdx.z, h = blockIdx.y, hk = h / (a.heads / a.heads_k);
  const SeqInfo si = seq_info(a.cu_seqlens_q, a.cu_seqlens_k, nullptr, nullptr, a.seqlen_q, a.seqlen_k,
                              a.use_mask_shift, a.mask_shift, b);
  // heaviest blocks (largest row index under a causal mask) first; with split-KV the splits of a row block are neighbours
  const int split = P.num_splits > 1 ? (int)blockIdx.x % P.num_splits : 0;
  const int mrank = P.num_splits > 1 ? (int)blockIdx.x / P.num_splits : (int)blockIdx.x;
  const int mblk = (int)gridDim.x / P.num_splits - 1 - mrank;
  const int m_base = mblk * C::NT * kBM;
  if (m_base >= si.sq) return;  // uniform for the CTA

  // per-tile key block ranges
  int lo[2], hi[2];
  bool active[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int m0 = m_base + t * kBM;
    active[t] = t < C::NT && m0 < si.sq;
    if (active[t]) {
      key_block_range(m0, kBM, kBN, si.sk, si.shift, a.window_left, a.window_right, lo[t], hi[t]);
      if (P.num_splits > 1) {
        lo[t] = max(lo[t], split * P.blocks_per_split);
        hi[t] = min(hi[t], (split + 1) * P.blocks_per_split);
        if (hi[t] <= lo[t]) lo[t] = hi[t] = 0;
      }
    } else {
      lo[t] = hi[t] = 0;
    }
  }
  int J_lo, J_hi;
  if (hi[0] > lo[0] && hi[1] > lo[1]) {
    J_lo = min(lo[0], lo[1]);
    J_hi = max(hi[0], hi[1]);
  } else if (hi[0] > lo[0]) {
    J_lo = lo[0];
    J_hi = hi[0];
  } else {
    J_lo = lo[1];
    J_hi = hi[1];
  }
  const int nblk = J_hi - J_lo;  // may be 0

  if (threadIdx.x == 0) {
    abort_init(abort_flag, P.status);
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_qfull(t), 1);
      mbar_init(bar_sfull(t), 1);
      mbar_init(bar_pfull(t), 4);
      mbar_init(bar_pfull_b(t), 4);
      mbar_init(bar_ofull(t), 1);
    }
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 10) {
    tmem_alloc(smem_addr(const_cast<uint32_t*>(tmem_ptr_smem)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_ptr_smem;

  const float scale_log2 = a.softmax_scale * kLog2e;

  if (warp < 8) {
    // ------------------------------------------------------------------ softmax warpgroups
    setmaxnreg_inc<216>();
    const int t = warp >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    const int row = m_base + t * kBM + row_in_tile;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_off + (t ? C::COL_S1 : C::COL_S0);
    const uint32_t tO = tmem + lane_off + (t ? C::COL_O1 : C::COL_O0);
    float m_used = -INFINITY;
    bool ok = true;
    // first / last visible key of this row (inclusive)
    int col_first = 0, col_last = si.sk - 1;
    if (a.window_right >= 0) col_last = min(col_last, row + si.shift + a.window_right);
    if (a.window_left >= 0) col_first = max(col_first, row + si.shift - a.window_left);
    const int m0 = m_base + t * kBM;

    const uint64_t scale2 = pack2(scale_log2, scale_log2);
    uint64_t l_sum2 = pack2(0.f, 0.f);  // two running partial row sums (even / odd columns)
    for (int j = lo[t]; j < hi[t] && ok; ++j) {
      const int it = j - lo[t];
      const bool first_block = it == 0;
      ok = mbar_wait(bar_sfull(t), it & 1, W_SFULL, abort_flag);
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
          if (!mbar_wait(bar_ofull(t), (it - 1) & 1, W_OFULL, abort_flag)) return false;
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
          if (lane == 0) mbar_arrive(half ? bar_pfull_b(t) : bar_pfull(t));
        }
        return true;
      };
      ok = need_mask ? block(std::true_type{}) : block(std::false_type{});
    }
    float l_sum;
    {
      float la, lb;
      unpack2(l_sum2, la, lb);
      l_sum = la + lb;
    }

    // ---- epilogue: O / l -> shared (swizzled) -> coalesced global stores; LSE
    if (active[t]) {
      const int n_it = hi[t] - lo[t];
      bool have_o = n_it > 0 && ok;
      if (have_o) {
        ok = mbar_wait(bar_ofull(t), (n_it - 1) & 1, W_OFULL, abort_flag);
        have_o = ok;
        tc_fence_after();
      }
      if (ok) {
        const bool empty = !(l_sum > 0.f) || m_used == -INFINITY;
        const float inv = empty ? 0.f : 1.f / l_sum;
        const float lse = empty ? INFINITY : (m_used + log2f(l_sum)) * kLn2;
        if (row < si.sq) {
          if (P.num_splits > 1)  // the split workspaces are (split, batch, head, row): not packed, -inf marks an empty part
            a.lse_accum[((int64_t)split * a.batch * a.heads + (int64_t)b * a.heads + h) * a.seqlen_q + row] = empty ? -INFINITY : lse;
          else
            a.softmax_lse[((int64_t)b * a.heads + h) * a.lse_seqlen + row] = lse;
        }
        unsigned char* stage = smem + t * C::TILE_BYTES;  // the Q tile of this warpgroup is no longer read
        constexpr int ROWB = DH * 2;
        // O leaves tensor memory 128 columns per round trip (a trip costs ~250 cycles whatever its size)
        constexpr int OB = DH < 128 ? DH : 128;
        uint32_t ob[OB / 32][32];
#pragma unroll
        for (int c0 = 0; c0 < DH; c0 += 32) {
          if (c0 % OB == 0) {
            if (have_o) {
#pragma unroll
              for (int c = 0; c < OB; c += 32) tmem_ld32(tO + c0 + c, ob[c / 32]);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int c = 0; c < OB / 32; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) ob[c][i] = 0u;
            }
          }
          const uint32_t(&o)[32] = ob[(c0 % OB) / 32];
          if (P.num_splits > 1) {  // normalised fp32 partial, straight from the registers (rows are contiguous)
            if (row < si.sq) {
              float* oa = a.out_accum +
                          (((int64_t)split * a.batch * a.heads + (int64_t)b * a.heads + h) * a.seqlen_q + row) * a.head_dim;
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                if (c0 + i < a.head_dim)
                  *reinterpret_cast<float4*>(oa + c0 + i) =
                      make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                                  __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            }
            continue;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {  // four 16-byte chunks of 8 elements
            uint4 pk;
            pk.x = Pack<T>::two(__uint_as_float(o[q4 * 8 + 0]) * inv, __uint_as_float(o[q4 * 8 + 1]) * inv);
            pk.y = Pack<T>::two(__uint_as_float(o[q4 * 8 + 2]) * inv, __uint_as_float(o[q4 * 8 + 3]) * inv);
            pk.z = Pack<T>::two(__uint_as_float(o[q4 * 8 + 4]) * inv, __uint_as_float(o[q4 * 8 + 5]) * inv);
            pk.w = Pack<T>::two(__uint_as_float(o[q4 * 8 + 6]) * inv, __uint_as_float(o[q4 * 8 + 7]) * inv);
            const int chunk = c0 / 8 + q4;
            const int phys = (chunk & ~7) | ((chunk ^ row_in_tile) & 7);
            *reinterpret_cast<uint4*>(stage + row_in_tile * ROWB + phys * 16) = pk;
          }
        }
      }
      named_bar_sync(1 + t, 128);
      if (ok && P.num_splits <= 1) {
        constexpr int CPR = DH / 8;  // 16-byte chunks per row
        const int tid = threadIdx.x & 127;
        unsigned char* stage = smem + t * C::TILE_BYTES;
        T* og = reinterpret_cast<T*>(a.out.ptr) + si.q_batch * a.out.stride_b + si.q_row0 * a.out.stride_s +
                (int64_t)h * a.out.stride_h;
#pragma unroll 4
        for (int i = tid; i < kBM * CPR; i += 128) {
          const int r = i / CPR, chunk = i % CPR;
          const int grow_ = m0 + r;
          if (grow_ < si.sq) {
            const int phys = (chunk & ~7) | ((chunk ^ r) & 7);
            uint4 v = *reinterpret_cast<const uint4*>(stage + r * (DH * 2) + phys * 16);
            if (chunk * 8 < a.head_dim) *reinterpret_cast<uint4*>(og + (int64_t)grow_ * a.out.stride_s + chunk * 8) = v;
          }
        }
      }
    }
  } else {
    setmaxnreg_dec<64>();
    if (warp == 8) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        const int qrow = (int)si.q_row0 + m_base;
        const int qb = (int)si.q_batch, kb = (int)si.k_batch;
        for (int t = 0; t < 2; ++t) {
          if (!active[t] || hi[t] <= lo[t]) continue;
          mbar_expect_tx(bar_qfull(t), C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c)
            tma_load_4d(sQ + t * C::TILE_BYTES + c * kChunkBytes, &P.tq, bar_qfull(t), c * 64, qrow + t * kBM, h, qb);
        }
        bool ok = true;
        for (int idx = 0; idx < 2 * nblk && ok; ++idx) {
          const int slot = idx % C::STAGES, round = idx / C::STAGES;
          ok = mbar_wait(bar_empty(slot), (round & 1) ^ 1, W_KVEMPTY, abort_flag);
          if (!ok) break;
          const int j = J_lo + (idx >> 1);
          const CUtensorMap* tm = (idx & 1) ? &P.tv : &P.tk;
          mbar_expect_tx(bar_full(slot), C::TILE_BYTES);
          for (int c = 0; c < C::NCHUNK; ++c)
            tma_load_4d(sKV + slot * C::TILE_BYTES + c * kChunkBytes, tm, bar_full(slot), c * 64,
                        (int)si.k_row0 + j * kBN, hk, kb);
        }
      }
    } else if (warp == 9) {
      // ---------------------------------------------------------------- MMA issuer
      {  // the whole warp runs the loop (see mma_ss_w); one elected lane issues
        constexpr uint32_t idesc_s = make_idesc(kBM, kBN, Fmt<T>::kIdesc, 0, 0);
        constexpr uint32_t idesc_o = make_idesc(kBM, DH, Fmt<T>::kIdesc, 0, 1);
        bool ok = true;
        int p_iter[2] = {0, 0};  // softmax iterations consumed per tile
        // One descriptor is built (Q tile 0, K-major); every other operand differs from it only in the
        // low word: the address field (+ byte offset >> 4) and, for MN-major reads, the LBO field.
        const uint64_t d_base = smem_desc_sw128(sQ, 16, 1024);
        const uint32_t d_lo = (uint32_t)d_base, d_hi = (uint32_t)(d_base >> 32);
        auto dsc = [&](uint32_t lo_add) { return ((uint64_t)d_hi << 32) | (uint64_t)(d_lo + lo_add); };
        constexpr uint32_t kMn = (uint32_t)((kChunkBytes - 16) >> 4) << 16;  // K-major -> MN-major (LBO = chunk stride)
        constexpr uint32_t kTile16 = C::TILE_BYTES >> 4, oKV = (C::NT * C::TILE_BYTES) >> 4;
        auto issue_s = [&](int t, int slot) {
          const uint32_t d = tmem + (t ? C::COL_S1 : C::COL_S0);
          const uint32_t a_lo = t ? kTile16 : 0u, b_lo = oKV + slot * kTile16;
#pragma unroll
          for (int kk = 0; kk < DH / 16; ++kk) {
            const uint32_t off = (uint32_t)(((kk >> 2) * kChunkBytes + (kk & 3) * 32) >> 4);
            mma_ss_w(d, dsc(a_lo + off), dsc(b_lo + off), idesc_s, kk > 0);
          }
          tc_commit_w(bar_sfull(t));
        };
        // PV in two halves of four k-steps: the softmax warps hand over P in two pieces (keys 0-63, then 64-127)
        auto issue_pv_half = [&](int t, int slot, bool first, int half) {
          const uint32_t d = tmem + (t ? C::COL_O1 : C::COL_O0);
          const uint32_t pa = tmem + (t ? C::COL_S1 : C::COL_S0);
          const uint32_t b_lo = oKV + slot * kTile16 + kMn;
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = half * 4 + k4;
            mma_ts_w(d, pa + kk * 8, dsc(b_lo + (uint32_t)((kk * 2048) >> 4)), idesc_o, (!first) || kk > 0);
          }
          if (half) tc_commit_w(bar_ofull(t));
        };
        auto in_range = [&](int t, int j) { return j >= lo[t] && j < hi[t]; };
        auto slot_of = [&](int idx) { return idx % C::STAGES; };
        auto par_of = [&](int idx) { return (uint32_t)((idx / C::STAGES) & 1); };
        // (Testing each barrier one MMA group ahead of its use, so that the answer travels while the group before
        // is being issued, was measured here and lost 3-5 %: the tests themselves take issue slots of this warp.)
        if (nblk > 0) {
          for (int t = 0; t < C::NT && ok; ++t)
            if (hi[t] > lo[t]) ok = mbar_wait_w(bar_qfull(t), 0, W_QFULL, abort_flag);
          // prologue: S_t(J_lo)
          if (ok) ok = mbar_wait_w(bar_full(slot_of(0)), par_of(0), W_KVFULL, abort_flag);
          if (ok) {
            tc_fence_after();
            for (int t = 0; t < C::NT; ++t)
              if (in_range(t, J_lo)) issue_s(t, slot_of(0));
            tc_commit_w(bar_empty(slot_of(0)));
          }
          for (int j = J_lo; j < J_hi && ok; ++j) {
            const int iv = 2 * (j - J_lo) + 1;  // ring index of V(j)
            const int ik = iv + 1;              // ring index of K(j+1)
            const bool more = j + 1 < J_hi;
            ok = mbar_wait_w(bar_full(slot_of(iv)), par_of(iv), W_KVFULL, abort_flag);
            if (ok && more) ok = mbar_wait_w(bar_full(slot_of(ik)), par_of(ik), W_KVFULL, abort_flag);
            if (!ok) break;
#pragma unroll
            for (int t = 0; t < C::NT; ++t) {
              if (!ok) break;
              if (in_range(t, j)) {
                const uint32_t par = (uint32_t)(p_iter[t] & 1);
                ok = mbar_wait_w(bar_pfull(t), par, W_PFULL, abort_flag);
                if (!ok) break;
                tc_fence_after();
                issue_pv_half(t, slot_of(iv), j == lo[t], 0);
                ok = mbar_wait_w(bar_pfull_b(t), par, W_PFULL, abort_flag);
                if (!ok) break;
                tc_fence_after();
                issue_pv_half(t, slot_of(iv), j == lo[t], 1);
                ++p_iter[t];
              }
              if (t == C::NT - 1) tc_commit_w(bar_empty(slot_of(iv)));
              if (more && in_range(t, j + 1)) issue_s(t, slot_of(ik));
              if (more && t == C::NT - 1) tc_commit_w(bar_empty(slot_of(ik)));
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
    // give copies that may still be in flight time to land before the shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == 10) tmem_dealloc(tmem, C::TMEM_COLS);
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
  P.num_splits = a.num_splits > 1 ? a.num_splits : 1;
  const int n_blocks = (a.seqlen_k + kBN - 1) / kBN;
  P.blocks_per_split = (n_blocks + P.num_splits - 1) / P.num_splits;
  auto kern = fwd_tc_kernel<T, DH>;
  static fa_host::DeviceOnce once;
  if (int rc = fa_host::raise_smem_limit(once, reinterpret_cast<const void*>(kern), C::SMEM_BYTES, "fwd_tc_kernel")) return rc;
  const int n_m = (a.seqlen_q + C::NT * kBM - 1) / (C::NT * kBM);
  dim3 grid(n_m * P.num_splits, a.heads, a.batch);
  kern<<<grid, 384, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("fwd_tc_kernel");
}

}  // namespace

bool fwd_tc_eligible(const FaFwdArgs& a) {
  if (a.head_dim > 256 || a.p_dropout > 0.f || a.s_dmask) return false;
  if (a.num_splits > 1 && a.cu_seqlens_q) return false;
  if (a.seqused_k || a.kv_batch_idx || a.block_table) return false;
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
