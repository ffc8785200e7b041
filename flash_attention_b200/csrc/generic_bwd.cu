// Any-shape backward attention (warp-level mma.sync path) plus the two bandwidth kernels that
// bracket every backward: rowsum(dO*O) and the fp32 -> 16-bit conversion of dQ.
//
// Structure follows the reference's three launches (csrc/flash_attn/src/flash_bwd_launch_template.h:47-90):
//   bwd_dot_do_o_kernel   D_i = sum_d dO_id O_id, and zero the fp32 dQ accumulator   (flash_bwd_kernel.h:106-186)
//   bwd_generic_kernel    one CTA per 64-key block: loop over query blocks, recompute
//                         P = exp2(S*scale_log2 - LSE*log2e), dV += P^T dO, dP = dO V^T,
//                         dS = P o (dP - D), dK += dS^T Q, dQ += dS K by fp32 atomics       (flash_bwd_kernel.h:425-1112)
//   bwd_convert_dq_kernel dQ = cast(dq_accum * softmax_scale)                              (flash_bwd_kernel.h:230-308)
// Differences by design: with grouped-query heads the CTA owns a KV head and walks all query
// heads of its group, so dK/dV need neither the expanded temporaries nor the group reduction of
// flash_api.cpp:744-751, 799-803, and stay free of atomics (bit-reproducible).  Head dims above
// 128 are handled by splitting the dK/dV/dQ columns over two CTAs that both contract over the
// full head dim.
#include "fa_common.cuh"

namespace fa {

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) bwd_dot_do_o_kernel(const __grid_constant__ FaBwdArgs p, const int zero_dq,
                                                           const int tpr_log2) {
  // Pure streaming: tpr = 2^tpr_log2 >= D/8 threads share a row, 16 bytes of O and of dO each; a CTA
  // covers kRows rows in passes of 256/tpr rows, four passes in flight per thread.  Grid
  // (ceil(max_sq/kRows), heads, batch).  zero_dq = 0 when the caller needs no cleared accumulator.
  constexpr int kRows = 128;
  const int tpr = 1 << tpr_log2;
  const int sub = threadIdx.x & (tpr - 1);       // which 16-byte piece of the row
  const int r_in_pass = threadIdx.x >> tpr_log2;  // row within a pass
  const int rows_per_pass = 256 >> tpr_log2;
  const int h = blockIdx.y, b = blockIdx.z;
  const SeqInfo si = seq_info(p.cu_seqlens_q, p.cu_seqlens_k, nullptr, nullptr, p.seqlen_q, p.seqlen_k,
                              p.use_mask_shift, p.mask_shift, b);
  const int D = p.head_dim;
  const int c = sub * 8;
  const bool col_ok = c < D;
  float* dsum = p.softmax_d + ((int64_t)b * p.heads + h) * p.d_seqlen;
  const T* obase = reinterpret_cast<const T*>(p.out.ptr) + si.q_batch * p.out.stride_b + (int64_t)h * p.out.stride_h + c;
  const T* dobase = reinterpret_cast<const T*>(p.dout.ptr) + si.q_batch * p.dout.stride_b + (int64_t)h * p.dout.stride_h + c;
  const int row0 = blockIdx.x * kRows;
  for (int base = 0; base < kRows; base += 4 * rows_per_pass) {
    uint4 a[4], d[4];
    int row[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      row[u] = row0 + base + u * rows_per_pass + r_in_pass;
      const bool ok = col_ok && row[u] < si.sq;
      a[u] = d[u] = make_uint4(0u, 0u, 0u, 0u);
      if (ok) {
        a[u] = *reinterpret_cast<const uint4*>(obase + (si.q_row0 + row[u]) * p.out.stride_s);
        d[u] = *reinterpret_cast<const uint4*>(dobase + (si.q_row0 + row[u]) * p.dout.stride_s);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float acc = Pack<T>::lo(a[u].x) * Pack<T>::lo(d[u].x) + Pack<T>::hi(a[u].x) * Pack<T>::hi(d[u].x);
      acc += Pack<T>::lo(a[u].y) * Pack<T>::lo(d[u].y) + Pack<T>::hi(a[u].y) * Pack<T>::hi(d[u].y);
      acc += Pack<T>::lo(a[u].z) * Pack<T>::lo(d[u].z) + Pack<T>::hi(a[u].z) * Pack<T>::hi(d[u].z);
      acc += Pack<T>::lo(a[u].w) * Pack<T>::lo(d[u].w) + Pack<T>::hi(a[u].w) * Pack<T>::hi(d[u].w);
      for (int o = tpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (sub == 0 && row[u] < p.d_seqlen) dsum[row[u]] = row[u] < si.sq ? acc : 0.f;
      if (zero_dq && col_ok && row[u] < si.sq) {
        // dq_accum is (batch, seqlen_q, heads, D) or packed (total_q, heads, D), fp32
        float* dqa = p.dq_accum + ((si.q_batch * (int64_t)p.seqlen_q + si.q_row0 + row[u]) * p.heads + h) * D + c;
        *reinterpret_cast<float4*>(dqa) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(dqa + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) bwd_convert_dq_kernel(const __grid_constant__ FaBwdArgs p) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int h = blockIdx.y, b = blockIdx.z;
  const SeqInfo si = seq_info(p.cu_seqlens_q, p.cu_seqlens_k, nullptr, nullptr, p.seqlen_q, p.seqlen_k,
                              p.use_mask_shift, p.mask_shift, b);
  if (row >= si.sq) return;
  const int D = p.head_dim;
  const float* dqa = p.dq_accum + ((si.q_batch * (int64_t)p.seqlen_q + si.q_row0 + row) * p.heads + h) * D;
  T* dq = reinterpret_cast<T*>(p.dq.ptr) + si.q_batch * p.dq.stride_b + (si.q_row0 + row) * p.dq.stride_s +
          (int64_t)h * p.dq.stride_h;
  const float sc = p.softmax_scale;
  for (int c = lane * 8; c < D; c += 256) {
    float4 x = *reinterpret_cast<const float4*>(dqa + c);
    float4 y = *reinterpret_cast<const float4*>(dqa + c + 4);
    uint4 o;
    o.x = Pack<T>::two(x.x * sc, x.y * sc);
    o.y = Pack<T>::two(x.z * sc, x.w * sc);
    o.z = Pack<T>::two(y.x * sc, y.y * sc);
    o.w = Pack<T>::two(y.z * sc, y.w * sc);
    *reinterpret_cast<uint4*>(dq + c) = o;
  }
}

template <typename T, int DP>
__device__ __forceinline__ void load_tile_64b(T* s, const T* g, int64_t row_stride, int row0, int nrows_valid, int D,
                                              int tid) {
  constexpr int CPR = DP / 8;
  for (int c = tid; c < 64 * CPR; c += 128) {
    int r = c / CPR, cc = (c % CPR) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    int gr = row0 + r;
    if (gr < nrows_valid && cc < D) val = *reinterpret_cast<const uint4*>(g + (int64_t)gr * row_stride + cc);
    *reinterpret_cast<uint4*>(s + r * (DP + 8) + cc) = val;
  }
}

// DP: padded head dim contracted over (64/128/256); DA = min(DP,128): columns of dK/dV/dQ that
// this CTA owns (column part = blockIdx.x % (DP/DA)).
template <typename T, int DP>
__global__ void __launch_bounds__(128) bwd_generic_kernel(const __grid_constant__ FaBwdArgs p, const int nblk0) {
  constexpr int DA = DP > 128 ? 128 : DP;
  constexpr int NPART = DP / DA;
  constexpr int LD = DP + 8;
  constexpr int LP = 64 + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sK = reinterpret_cast<T*>(smem_raw);
  T* sV = sK + 64 * LD;
  T* sQ = sV + 64 * LD;
  T* sdO = sQ + 64 * LD;
  T* sP = sdO + 64 * LD;
  T* sdS = sP + 64 * LP;
  float* sLse = reinterpret_cast<float*>(sdS + 64 * LP);
  float* sD = sLse + 64;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int part = blockIdx.x % NPART;
  const int nblk = nblk0 + blockIdx.x / NPART;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.heads / p.heads_k;
  const SeqInfo si = seq_info(p.cu_seqlens_q, p.cu_seqlens_k, nullptr, nullptr, p.seqlen_q, p.seqlen_k,
                              p.use_mask_shift, p.mask_shift, b);
  const int n0 = nblk * 64;
  if (n0 >= si.sk) return;
  const int D = p.head_dim;
  const int dcol0 = part * DA;
  const T* kg = reinterpret_cast<const T*>(p.k.ptr) + si.k_batch * p.k.stride_b + si.k_row0 * p.k.stride_s +
                (int64_t)hk * p.k.stride_h;
  const T* vg = reinterpret_cast<const T*>(p.v.ptr) + si.k_batch * p.v.stride_b + si.k_row0 * p.v.stride_s +
                (int64_t)hk * p.v.stride_h;
  load_tile_64b<T, DP>(sK, kg, p.k.stride_s, n0, si.sk, D, tid);
  load_tile_64b<T, DP>(sV, vg, p.v.stride_s, n0, si.sk, D, tid);

  float dk_acc[DA / 8][4], dv_acc[DA / 8][4];
#pragma unroll
  for (int i = 0; i < DA / 8; ++i) {
    dk_acc[i][0] = dk_acc[i][1] = dk_acc[i][2] = dk_acc[i][3] = 0.f;
    dv_acc[i][0] = dv_acc[i][1] = dv_acc[i][2] = dv_acc[i][3] = 0.f;
  }
  const float scale_log2 = p.softmax_scale * kLog2e;
  const bool do_drop = p.p_dropout > 0.f;
  const uint32_t keep_thr = (uint32_t)floorf((1.f - p.p_dropout) * 255.f);
  const float rp_keep = do_drop ? 1.f / (1.f - p.p_dropout) : 1.f;

  int m_lo, m_hi;
  query_block_range(n0, 64, 64, si.sq, si.shift, p.window_left, p.window_right, m_lo, m_hi);

  for (int hq = hk * group; hq < (hk + 1) * group; ++hq) {
    const int bh = b * p.heads + hq;
    const T* qg = reinterpret_cast<const T*>(p.q.ptr) + si.q_batch * p.q.stride_b + si.q_row0 * p.q.stride_s +
                  (int64_t)hq * p.q.stride_h;
    const T* dog = reinterpret_cast<const T*>(p.dout.ptr) + si.q_batch * p.dout.stride_b +
                   si.q_row0 * p.dout.stride_s + (int64_t)hq * p.dout.stride_h;
    const float* lse_g = p.softmax_lse + (int64_t)bh * p.lse_seqlen;
    const float* d_g = p.softmax_d + (int64_t)bh * p.d_seqlen;
    for (int m = m_lo; m < m_hi; ++m) {
      const int m0 = m * 64;
      __syncthreads();  // everyone is done with the previous Q/dO/P/dS tiles
      load_tile_64b<T, DP>(sQ, qg, p.q.stride_s, m0, si.sq, D, tid);
      load_tile_64b<T, DP>(sdO, dog, p.dout.stride_s, m0, si.sq, D, tid);
      if (tid < 64) {
        int r = m0 + tid;
        sLse[tid] = r < si.sq ? lse_g[r] : INFINITY;
        sD[tid] = r < si.sq ? d_g[r] : 0.f;
      }
      __syncthreads();

      // S = Q K^T and dP = dO V^T for this warp's 16 query rows x 64 keys
      float s[8][4], dp[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < DP / 16; ++ks) {
        uint32_t aq[4], ado[4];
        const int arow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, acol = ks * 16 + (lane >> 4) * 8;
        ldsm_x4(aq, smem_u32(sQ + arow * LD + acol));
        ldsm_x4(ado, smem_u32(sdO + arow * LD + acol));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bk[4], bv[4];
          const int brow = np * 16 + (lane & 7) + (lane >> 4) * 8, bcol = ks * 16 + ((lane >> 3) & 1) * 8;
          ldsm_x4(bk, smem_u32(sK + brow * LD + bcol));
          ldsm_x4(bv, smem_u32(sV + brow * LD + bcol));
          mma16816<T>(s[2 * np], aq, bk[0], bk[1]);
          mma16816<T>(s[2 * np + 1], aq, bk[2], bk[3]);
          mma16816<T>(dp[2 * np], ado, bv[0], bv[1]);
          mma16816<T>(dp[2 * np + 1], ado, bv[2], bv[3]);
        }
      }
      // P, dS -> shared (16-bit), in [query][key] order
      const int lr = warp * 16 + g;
      const float lse_log2[2] = {sLse[lr] * kLog2e, sLse[lr + 8] * kLog2e};
      const float dsum[2] = {sD[lr], sD[lr + 8]};
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint4 blk = make_uint4(0, 0, 0, 0);
        if (do_drop) blk = dropout_block(p.rng_seed, p.rng_offset, bh, (m0 + warp * 16) >> 4, (n0 >> 5) + cb, lane);
#pragma unroll
        for (int n4 = 0; n4 < 4; ++n4) {
          const int nt = cb * 4 + n4;
          float pv[4], dsv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            int col = n0 + nt * 8 + 2 * t + (e & 1);
            int row = m0 + lr + (e >> 1) * 8;
            bool vis = row < si.sq && visible(row, col, si.sk, si.shift, p.window_left, p.window_right);
            float pe = vis ? fast_exp2(s[nt][e] * scale_log2 - lse_log2[e >> 1]) : 0.f;
            bool keep = !do_drop || dropout_byte_of(blk, e >> 1, n4, e & 1) <= keep_thr;
            float dpe = keep ? dp[nt][e] * rp_keep : 0.f;
            dsv[e] = pe * (dpe - dsum[e >> 1]);
            pv[e] = keep ? pe * rp_keep : 0.f;
          }
          const int c = nt * 8 + 2 * t;
          *reinterpret_cast<uint32_t*>(sP + lr * LP + c) = Pack<T>::two(pv[0], pv[1]);
          *reinterpret_cast<uint32_t*>(sP + (lr + 8) * LP + c) = Pack<T>::two(pv[2], pv[3]);
          *reinterpret_cast<uint32_t*>(sdS + lr * LP + c) = Pack<T>::two(dsv[0], dsv[1]);
          *reinterpret_cast<uint32_t*>(sdS + (lr + 8) * LP + c) = Pack<T>::two(dsv[2], dsv[3]);
        }
      }
      __syncthreads();

      // dV[16 keys of this warp, DA cols] += P^T dO ; dK += dS^T Q
#pragma unroll
      for (int kq = 0; kq < 4; ++kq) {  // 16 query rows per k-step
        uint32_t ap[4], ads[4];
        const int prow = kq * 16 + (lane & 7) + (lane >> 4) * 8, pcol = warp * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4_t(ap, smem_u32(sP + prow * LP + pcol));
        ldsm_x4_t(ads, smem_u32(sdS + prow * LP + pcol));
#pragma unroll
        for (int dt = 0; dt < DA / 16; ++dt) {
          uint32_t bdo[4], bq[4];
          const int brow = kq * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, bcol = dcol0 + dt * 16 + (lane >> 4) * 8;
          ldsm_x4_t(bdo, smem_u32(sdO + brow * LD + bcol));
          ldsm_x4_t(bq, smem_u32(sQ + brow * LD + bcol));
          mma16816<T>(dv_acc[2 * dt], ap, bdo[0], bdo[1]);
          mma16816<T>(dv_acc[2 * dt + 1], ap, bdo[2], bdo[3]);
          mma16816<T>(dk_acc[2 * dt], ads, bq[0], bq[1]);
          mma16816<T>(dk_acc[2 * dt + 1], ads, bq[2], bq[3]);
        }
      }
      // dQ[16 rows of this warp, DA cols] = dS K, 64 columns at a time, fp32 atomics
      float* dqa = p.dq_accum + ((si.q_batch * (int64_t)p.seqlen_q + si.q_row0) * p.heads + hq) * D;
      const int64_t dq_rs = (int64_t)p.heads * D;
#pragma unroll
      for (int dc = 0; dc < DA / 64; ++dc) {
        float dq[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 keys per k-step
          uint32_t a[4];
          ldsm_x4(a, smem_u32(sdS + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LP + kk * 16 + (lane >> 4) * 8));
#pragma unroll
          for (int dt = 0; dt < 4; ++dt) {
            uint32_t bb[4];
            ldsm_x4_t(bb, smem_u32(sK + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dcol0 + dc * 64 + dt * 16 +
                                   (lane >> 4) * 8));
            mma16816<T>(dq[2 * dt], a, bb[0], bb[1]);
            mma16816<T>(dq[2 * dt + 1], a, bb[2], bb[3]);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          int col = dcol0 + dc * 64 + i * 8 + 2 * t;
          if (col < D) {
            int r0 = m0 + lr, r1 = r0 + 8;
            if (r0 < si.sq) {
              atomicAdd(dqa + r0 * dq_rs + col, dq[i][0]);
              atomicAdd(dqa + r0 * dq_rs + col + 1, dq[i][1]);
            }
            if (r1 < si.sq) {
              atomicAdd(dqa + r1 * dq_rs + col, dq[i][2]);
              atomicAdd(dqa + r1 * dq_rs + col + 1, dq[i][3]);
            }
          }
        }
      }
    }
  }

  // epilogue: dK (scaled) and dV for keys n0 + warp*16 + {g, g+8}
  const int kr0 = n0 + warp * 16 + g;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    int krow = kr0 + r * 8;
    if (krow >= si.sk) continue;
    if (p.accumulate_dkv) {
      float* dka = p.dk_accum + ((si.k_batch * (int64_t)p.seqlen_k + si.k_row0 + krow) * p.heads_k + hk) * D;
      float* dva = p.dv_accum + ((si.k_batch * (int64_t)p.seqlen_k + si.k_row0 + krow) * p.heads_k + hk) * D;
#pragma unroll
      for (int i = 0; i < DA / 8; ++i) {
        int col = dcol0 + i * 8 + 2 * t;
        if (col < D) {
          float2 a = *reinterpret_cast<float2*>(dka + col), c = *reinterpret_cast<float2*>(dva + col);
          a.x += dk_acc[i][2 * r] * p.softmax_scale;
          a.y += dk_acc[i][2 * r + 1] * p.softmax_scale;
          c.x += dv_acc[i][2 * r];
          c.y += dv_acc[i][2 * r + 1];
          *reinterpret_cast<float2*>(dka + col) = a;
          *reinterpret_cast<float2*>(dva + col) = c;
        }
      }
    } else {
      T* dk = reinterpret_cast<T*>(p.dk.ptr) + si.k_batch * p.dk.stride_b + (si.k_row0 + krow) * p.dk.stride_s +
              (int64_t)hk * p.dk.stride_h;
      T* dv = reinterpret_cast<T*>(p.dv.ptr) + si.k_batch * p.dv.stride_b + (si.k_row0 + krow) * p.dv.stride_s +
              (int64_t)hk * p.dv.stride_h;
#pragma unroll
      for (int i = 0; i < DA / 8; ++i) {
        int col = dcol0 + i * 8 + 2 * t;
        if (col < D) {
          *reinterpret_cast<uint32_t*>(dk + col) =
              Pack<T>::two(dk_acc[i][2 * r] * p.softmax_scale, dk_acc[i][2 * r + 1] * p.softmax_scale);
          *reinterpret_cast<uint32_t*>(dv + col) = Pack<T>::two(dv_acc[i][2 * r], dv_acc[i][2 * r + 1]);
        }
      }
    }
  }
}

template <typename T, int DP>
static int launch_bwd_generic(const FaBwdArgs& a, cudaStream_t st) {
  size_t smem = (4 * 64 * (DP + 8) + 2 * 64 * 72) * sizeof(T) + 128 * sizeof(float);
  auto kern = bwd_generic_kernel<T, DP>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  constexpr int NPART = DP > 128 ? DP / 128 : 1;
  const int nblocks = (a.seqlen_k + 63) / 64;
  if (a.deterministic) {
    // One launch per key block: inside a launch no two CTAs add into the same dq value (they own different
    // batch entries, heads or column parts), and the stream orders the launches, so every dq value receives
    // its terms in key order.
    for (int nb = 0; nb < nblocks; ++nb) {
      kern<<<dim3(NPART, a.heads_k, a.batch), 128, smem, st>>>(a, nb);
      if (int rc = fa_host::check_launch("bwd_generic_kernel")) return rc;
    }
    return 0;
  }
  dim3 grid(nblocks * NPART, a.heads_k, a.batch);
  kern<<<grid, 128, smem, st>>>(a, 0);
  return fa_host::check_launch("bwd_generic_kernel");
}

template <typename T>
int bwd_pre_t(const FaBwdArgs& a, int zero_dq, cudaStream_t st) {
  int rows = a.d_seqlen > a.seqlen_q ? a.d_seqlen : a.seqlen_q;
  int tpr_log2 = 0;
  while ((8 << tpr_log2) < a.head_dim) ++tpr_log2;  // threads per row: a power of two >= head_dim / 8 (<= 32)
  dim3 grid((rows + 127) / 128, a.heads, a.batch);
  bwd_dot_do_o_kernel<T><<<grid, 256, 0, st>>>(a, zero_dq, tpr_log2);
  return fa_host::check_launch("bwd_dot_do_o_kernel");
}
template <typename T>
int bwd_post_t(const FaBwdArgs& a, cudaStream_t st) {
  dim3 grid((a.seqlen_q + 3) / 4, a.heads, a.batch);
  bwd_convert_dq_kernel<T><<<grid, 128, 0, st>>>(a);
  return fa_host::check_launch("bwd_convert_dq_kernel");
}

int bwd_pre(const FaBwdArgs& a, int zero_dq, cudaStream_t st) {
  return a.dtype == FA_DTYPE_BF16 ? bwd_pre_t<__nv_bfloat16>(a, zero_dq, st) : bwd_pre_t<__half>(a, zero_dq, st);
}
int bwd_post(const FaBwdArgs& a, cudaStream_t st) {
  return a.dtype == FA_DTYPE_BF16 ? bwd_post_t<__nv_bfloat16>(a, st) : bwd_post_t<__half>(a, st);
}

template <typename T>
static int dispatch_bwd_generic(const FaBwdArgs& a, cudaStream_t st) {
  if (a.head_dim <= 64) return launch_bwd_generic<T, 64>(a, st);
  if (a.head_dim <= 128) return launch_bwd_generic<T, 128>(a, st);
  return launch_bwd_generic<T, 256>(a, st);
}

int bwd_generic_main(const FaBwdArgs& a, cudaStream_t st) {
  return a.dtype == FA_DTYPE_BF16 ? dispatch_bwd_generic<__nv_bfloat16>(a, st) : dispatch_bwd_generic<__half>(a, st);
}

}  // namespace fa
