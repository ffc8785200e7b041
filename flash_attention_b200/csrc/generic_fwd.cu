// Any-shape forward attention kernel (warp-level mma.sync path).
//
// Covers what the tcgen05 kernels do not: head dims that are not 64/128, dropout, split-KV of
// long query blocks, operands whose strides or alignment rule out TMA.  One CTA = 64 query rows
// of one (batch, head) [x one KV split]; 4 warps of 16 rows; K/V streamed in 64-row tiles.
// Math follows compute_attn_1rowblock (csrc/flash_attn/src/flash_fwd_kernel.h:74-580): online
// softmax in the exp2 domain, O rescaled per tile, O /= rowsum and LSE = max*scale + log(sum) at
// the end, O = 0 / LSE = +inf for rows that see no key.
#include "fa_common.cuh"

namespace fa {

constexpr int GF_BM = 64;
constexpr int GF_BN = 64;

template <typename T, int DP>
__device__ __forceinline__ void load_tile_64(T* s, const T* g, int64_t row_stride, int row0, int nrows_valid, int D,
                                             int tid) {
  // copies rows [row0, row0+64) x cols [0, DP) of g into s[64][DP+8], zero-filling outside
  // (row < nrows_valid, col < D)
  constexpr int CPR = DP / 8;  // 16-byte chunks per row
  for (int c = tid; c < 64 * CPR; c += 128) {
    int r = c / CPR, cc = (c % CPR) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    int gr = row0 + r;
    if (gr < nrows_valid && cc < D) val = *reinterpret_cast<const uint4*>(g + (int64_t)gr * row_stride + cc);
    *reinterpret_cast<uint4*>(s + r * (DP + 8) + cc) = val;
  }
}

template <typename T, int DP>
__global__ void __launch_bounds__(128) fwd_generic_kernel(const __grid_constant__ FaFwdArgs p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + 64 * (DP + 8);
  T* sV = sK + 64 * (DP + 8);
  constexpr int LD = DP + 8;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int nsplit = p.num_splits > 1 ? p.num_splits : 1;
  const int b = blockIdx.z / nsplit, split = blockIdx.z % nsplit;
  const int h = blockIdx.y, hk = h / (p.heads / p.heads_k);
  const SeqInfo si = seq_info(p.cu_seqlens_q, p.cu_seqlens_k, p.seqused_k, p.kv_batch_idx, p.seqlen_q, p.seqlen_k,
                              p.use_mask_shift, p.mask_shift, b, p.seqused_k_extra);
  const int m0 = blockIdx.x * GF_BM;
  if (m0 >= si.sq) return;
  const int D = p.head_dim;
  const T* qg = reinterpret_cast<const T*>(p.q.ptr) + si.q_batch * p.q.stride_b + si.q_row0 * p.q.stride_s +
                (int64_t)h * p.q.stride_h;
  const int64_t kbatch = p.block_table ? 0 : si.k_batch;  // paged: the page offset is added per tile
  const T* kg = reinterpret_cast<const T*>(p.k.ptr) + kbatch * p.k.stride_b + si.k_row0 * p.k.stride_s +
                (int64_t)hk * p.k.stride_h;
  const T* vg = reinterpret_cast<const T*>(p.v.ptr) + kbatch * p.v.stride_b + si.k_row0 * p.v.stride_s +
                (int64_t)hk * p.v.stride_h;

  int n_lo, n_hi;
  key_block_range(m0, GF_BM, GF_BN, si.sk, si.shift, p.window_left, p.window_right, n_lo, n_hi);
  if (nsplit > 1) {
    int nb = (si.sk + GF_BN - 1) / GF_BN;
    int per = (nb + nsplit - 1) / nsplit;
    n_lo = max(n_lo, split * per);
    n_hi = min(n_hi, (split + 1) * per);
    if (n_hi < n_lo) n_hi = n_lo;
  }

  load_tile_64<T, DP>(sQ, qg, p.q.stride_s, m0, si.sq, D, tid);

  float o_acc[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float scale_log2 = p.softmax_scale * kLog2e;
  const bool do_drop = p.p_dropout > 0.f;
  const uint32_t keep_thr = (uint32_t)floorf((1.f - p.p_dropout) * 255.f);
  const int bh = b * p.heads + h;
  const int row_a = m0 + warp * 16 + g;  // rows row_a and row_a + 8

  for (int n = n_lo; n < n_hi; ++n) {
    const int n0 = n * GF_BN;
    __syncthreads();  // previous tile fully consumed (and sQ visible on the first pass)
    if (p.block_table) {
      // a 64-key tile never straddles a page (page_block_size % 64 == 0): rebase on the page the table names
      const int64_t page = p.block_table[(int64_t)b * p.block_table_stride + n0 / p.page_block_size];
      const int r0 = n0 % p.page_block_size;
      load_tile_64<T, DP>(sK, kg + page * p.k.stride_b, p.k.stride_s, r0, r0 + (si.sk - n0), D, tid);
      load_tile_64<T, DP>(sV, vg + page * p.v.stride_b, p.v.stride_s, r0, r0 + (si.sk - n0), D, tid);
    } else {
      load_tile_64<T, DP>(sK, kg, p.k.stride_s, n0, si.sk, D, tid);
      load_tile_64<T, DP>(sV, vg, p.v.stride_s, n0, si.sk, D, tid);
    }
    __syncthreads();

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < DP / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a, smem_u32(sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bb[4];
        ldsm_x4(bb, smem_u32(sK + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8));
        mma16816<T>(s[2 * np], a, bb[0], bb[1]);
        mma16816<T>(s[2 * np + 1], a, bb[2], bb[3]);
      }
    }
    // scale, mask, running max
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int col = n0 + nt * 8 + 2 * t + (e & 1);
        int row = row_a + (e >> 1) * 8;
        float x = visible(row, col, si.sk, si.shift, p.window_left, p.window_right) ? s[nt][e] * scale_log2 : -INFINITY;
        s[nt][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    float alpha[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      float mn = fmaxf(m_run[r], mx[r]);
      msafe[r] = mn == -INFINITY ? 0.f : mn;
      alpha[r] = fast_exp2(m_run[r] - msafe[r]);
      m_run[r] = mn;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      o_acc[i][0] *= alpha[0];
      o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1];
      o_acc[i][3] *= alpha[1];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float pv = fast_exp2(s[nt][e] - msafe[e >> 1]);
        l_run[e >> 1] += pv;
        s[nt][e] = pv;
      }
    if (do_drop) {
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {  // two 32-column dropout tiles per 64-column key tile
        uint4 blk = dropout_block(p.rng_seed, p.rng_offset, bh, (m0 + warp * 16) >> 4, (n0 >> 5) + cb, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (dropout_byte_of(blk, e >> 1, nt, e & 1) > keep_thr) s[cb * 4 + nt][e] = 0.f;
      }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = Pack<T>::two(s[2 * kk][0], s[2 * kk][1]);
      a[1] = Pack<T>::two(s[2 * kk][2], s[2 * kk][3]);
      a[2] = Pack<T>::two(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = Pack<T>::two(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dt = 0; dt < DP / 16; ++dt) {
        uint32_t bb[4];
        ldsm_x4_t(bb, smem_u32(sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dt * 16 + (lane >> 4) * 8));
        mma16816<T>(o_acc[2 * dt], a, bb[0], bb[1]);
        mma16816<T>(o_acc[2 * dt + 1], a, bb[2], bb[3]);
      }
    }
  }

  // epilogue
  float inv[2], lse[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    bool empty = !(l > 0.f) || m_run[r] == -INFINITY;
    inv[r] = empty ? 0.f : 1.f / l;
    lse[r] = empty ? INFINITY : (m_run[r] + log2f(l)) * kLn2;
  }
  const float rp_keep = do_drop ? 1.f / (1.f - p.p_dropout) : 1.f;
  if (nsplit > 1) {
    // partial results: normalised O in fp32 and LSE (-inf for an empty split)
    const int64_t rows_total = (int64_t)p.batch * p.heads * p.seqlen_q;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int row = row_a + r * 8;
      if (row >= si.sq) continue;
      int64_t ridx = ((int64_t)bh * p.seqlen_q + row);
      float* oa = p.out_accum + ((int64_t)split * rows_total + ridx) * D;
      if (t == 0) p.lse_accum[(int64_t)split * rows_total + ridx] = lse[r] == INFINITY ? -INFINITY : lse[r];
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        int col = i * 8 + 2 * t;
        if (col < D) *reinterpret_cast<float2*>(oa + col) = make_float2(o_acc[i][2 * r] * inv[r], o_acc[i][2 * r + 1] * inv[r]);
      }
    }
  } else {
    T* og = reinterpret_cast<T*>(p.out.ptr) + si.q_batch * p.out.stride_b + si.q_row0 * p.out.stride_s +
            (int64_t)h * p.out.stride_h;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int row = row_a + r * 8;
      if (row >= si.sq) continue;
      if (t == 0) p.softmax_lse[(int64_t)bh * p.lse_seqlen + row] = lse[r];
      float sc = inv[r] * rp_keep;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        int col = i * 8 + 2 * t;
        if (col < D)
          *reinterpret_cast<uint32_t*>(og + (int64_t)row * p.out.stride_s + col) =
              Pack<T>::two(o_acc[i][2 * r] * sc, o_acc[i][2 * r + 1] * sc);
      }
    }
  }
}

// Softmax probabilities with the dropout pattern in the sign bit, for return_softmax
// (flash_api.cpp:351-354).  The reference writes un-normalised tiles in its mma fragment order
// (flash_fwd_kernel.h:57-70); this build returns the normalised matrix exp(scale*q.k - lse) in
// plain (row, col) order, negative where dropped, zero where masked.
template <typename T>
__global__ void probs_kernel(const __grid_constant__ FaFwdArgs p) {
  const int b = blockIdx.z, h = blockIdx.y, hk = h / (p.heads / p.heads_k);
  const SeqInfo si = seq_info(p.cu_seqlens_q, p.cu_seqlens_k, p.seqused_k, p.kv_batch_idx, p.seqlen_q, p.seqlen_k,
                              p.use_mask_shift, p.mask_shift, b, p.seqused_k_extra);
  const int row = blockIdx.x;
  const int bh = b * p.heads + h;
  T* out = reinterpret_cast<T*>(p.s_dmask) + ((int64_t)bh * p.sdmask_rows + row) * p.sdmask_cols;
  if (row >= si.sq) {
    for (int j = threadIdx.x; j < p.sdmask_cols; j += blockDim.x) out[j] = Pack<T>::from(0.f);
    return;
  }
  extern __shared__ float sq[];
  const T* qg = reinterpret_cast<const T*>(p.q.ptr) + si.q_batch * p.q.stride_b + (si.q_row0 + row) * p.q.stride_s +
                (int64_t)h * p.q.stride_h;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) sq[d] = Pack<T>::one(qg[d]);
  __syncthreads();
  const T* kg = reinterpret_cast<const T*>(p.k.ptr) + si.k_batch * p.k.stride_b + si.k_row0 * p.k.stride_s +
                (int64_t)hk * p.k.stride_h;
  const float lse = p.softmax_lse[(int64_t)bh * p.lse_seqlen + row];
  const uint32_t keep_thr = (uint32_t)floorf((1.f - p.p_dropout) * 255.f);
  for (int j = threadIdx.x; j < p.sdmask_cols; j += blockDim.x) {
    float val = 0.f;
    if (visible(row, j, si.sk, si.shift, p.window_left, p.window_right)) {
      const T* kr = kg + (int64_t)j * p.k.stride_s;
      float acc = 0.f;
      for (int d = 0; d < p.head_dim; ++d) acc += sq[d] * Pack<T>::one(kr[d]);
      val = lse == INFINITY ? 0.f : __expf(acc * p.softmax_scale - lse);
      if (p.p_dropout > 0.f && dropout_byte(p.rng_seed, p.rng_offset, bh, row, j) > keep_thr) val = -val;
    }
    out[j] = Pack<T>::from(val);
  }
}

template <typename T, int DP>
static int launch_fwd_generic(const FaFwdArgs& a, cudaStream_t st) {
  size_t smem = 3 * 64 * (DP + 8) * sizeof(T);
  auto kern = fwd_generic_kernel<T, DP>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int nsplit = a.num_splits > 1 ? a.num_splits : 1;
  dim3 grid((a.seqlen_q + GF_BM - 1) / GF_BM, a.heads, a.batch * nsplit);
  kern<<<grid, 128, smem, st>>>(a);
  return fa_host::check_launch("fwd_generic_kernel");
}

template <typename T>
static int dispatch_fwd_generic(const FaFwdArgs& a, cudaStream_t st) {
  int rc;
  if (a.head_dim <= 64)
    rc = launch_fwd_generic<T, 64>(a, st);
  else if (a.head_dim <= 128)
    rc = launch_fwd_generic<T, 128>(a, st);
  else
    rc = launch_fwd_generic<T, 256>(a, st);
  if (rc) return rc;
  if (a.s_dmask && a.num_splits <= 1) {
    dim3 grid(a.sdmask_rows, a.heads, a.batch);
    probs_kernel<T><<<grid, 128, a.head_dim * sizeof(float), st>>>(a);
    return fa_host::check_launch("probs_kernel");
  }
  return 0;
}

int fwd_generic(const FaFwdArgs& a, cudaStream_t st) {
  return a.dtype == FA_DTYPE_BF16 ? dispatch_fwd_generic<__nv_bfloat16>(a, st) : dispatch_fwd_generic<__half>(a, st);
}

}  // namespace fa
