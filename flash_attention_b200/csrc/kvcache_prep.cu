// KV-cache append + rotary embedding as a stand-alone launch, used when a decode call does not fit
// the fused single-token kernel (several new tokens, long query blocks, odd head dims).
// Same effect as the prologue of compute_attn_1rowblock_splitkv
// (csrc/flash_attn/src/flash_fwd_kernel.h:768-891): new K rows are rotated at absolute position
// cache_seqlens[b] + i and written with the new V rows into the cache at batch slot
// cache_batch_idx[b]; q is rotated at cache_seqlens[b] + i when the mask is causal/local and at
// cache_seqlens[b] for every row otherwise.  Rotary math is fp32, rounded once
// (csrc/flash_attn/src/utils.h:391-517).
#include "fa_common.cuh"

namespace fa {

template <typename T>
__device__ __forceinline__ void rotate_row(const T* src, T* dst, const T* cosr, const T* sinr, int D, int rdim,
                                           bool interleaved, int lane_step, int lane0) {
  // cosr/sinr: row of rdim/2 values, or nullptr for a plain copy
  const int half = rdim / 2;
  for (int d = lane0; d < D; d += lane_step) {
    float x = Pack<T>::one(src[d]);
    float y = x;
    if (cosr && d < rdim) {
      int i, partner;
      bool first;
      if (interleaved) {
        i = d >> 1;
        first = (d & 1) == 0;
        partner = first ? d + 1 : d - 1;
      } else {
        first = d < half;
        i = first ? d : d - half;
        partner = first ? d + half : d - half;
      }
      float c = Pack<T>::one(cosr[i]), s = Pack<T>::one(sinr[i]);
      float xp = Pack<T>::one(src[partner]);
      y = first ? x * c - xp * s : x * c + xp * s;
    }
    dst[d] = Pack<T>::from(y);
  }
}

// grid: (seqlen_new + seqlen_q, max(heads, heads_k), batch); block 128
template <typename T>
__global__ void __launch_bounds__(128) kvcache_prep_kernel(const __grid_constant__ FaKvcacheArgs p, int q_follows_rows) {
  const int b = blockIdx.z, hh = blockIdx.y;
  const int L = p.cache_seqlens ? p.cache_seqlens[b] : p.seqlen_cache;
  const T* cosb = reinterpret_cast<const T*>(p.rotary_cos);
  const T* sinb = reinterpret_cast<const T*>(p.rotary_sin);
  const int half = p.rotary_dim / 2;
  const int D = p.head_dim;
  int r = blockIdx.x;
  if (r < p.seqlen_new) {
    if (hh >= p.heads_k || !p.knew.ptr) return;
    const int pos = L + r;
    if (pos >= p.seqlen_cache) return;
    int64_t cb = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
    int row = pos;
    if (p.block_table) {  // paged cache: the table names the page, the row is the position inside it
      cb = p.block_table[(int64_t)b * p.block_table_stride + pos / p.page_block_size];
      row = pos % p.page_block_size;
    }
    const T* ks = reinterpret_cast<const T*>(p.knew.ptr) + b * p.knew.stride_b + r * p.knew.stride_s + hh * p.knew.stride_h;
    const T* vs = reinterpret_cast<const T*>(p.vnew.ptr) + b * p.vnew.stride_b + r * p.vnew.stride_s + hh * p.vnew.stride_h;
    T* kd = reinterpret_cast<T*>(p.kcache.ptr) + cb * p.kcache.stride_b + (int64_t)row * p.kcache.stride_s + hh * p.kcache.stride_h;
    T* vd = reinterpret_cast<T*>(p.vcache.ptr) + cb * p.vcache.stride_b + (int64_t)row * p.vcache.stride_s + hh * p.vcache.stride_h;
    const bool rot = cosb != nullptr && pos < p.seqlen_ro;
    rotate_row<T>(ks, kd, rot ? cosb + (int64_t)pos * half : nullptr, rot ? sinb + (int64_t)pos * half : nullptr, D,
                  p.rotary_dim, p.rotary_interleaved != 0, blockDim.x, threadIdx.x);
    for (int d = threadIdx.x; d < D; d += blockDim.x) vd[d] = vs[d];
  } else {
    r -= p.seqlen_new;
    if (hh >= p.heads || !p.q_rotated || r >= p.seqlen_q) return;
    const int pos = L + (q_follows_rows ? r : 0);
    const T* qs = reinterpret_cast<const T*>(p.q.ptr) + b * p.q.stride_b + r * p.q.stride_s + hh * p.q.stride_h;
    // q_rotated is contiguous (batch, seqlen_q, heads, D)
    T* qd = reinterpret_cast<T*>(p.q_rotated) + (((int64_t)b * p.seqlen_q + r) * p.heads + hh) * D;
    const bool rot = cosb != nullptr && pos < p.seqlen_ro;
    rotate_row<T>(qs, qd, rot ? cosb + (int64_t)pos * half : nullptr, rot ? sinb + (int64_t)pos * half : nullptr, D,
                  p.rotary_dim, p.rotary_interleaved != 0, blockDim.x, threadIdx.x);
  }
}

int kvcache_prep(const FaKvcacheArgs& a, int q_follows_rows, cudaStream_t st) {
  int rows = (a.knew.ptr ? a.seqlen_new : 0);
  FaKvcacheArgs c = a;
  if (!a.knew.ptr) c.seqlen_new = 0;
  if (a.q_rotated) rows += a.seqlen_q;
  if (rows == 0) return 0;
  dim3 grid(rows, a.heads > a.heads_k ? a.heads : a.heads_k, a.batch);
  if (a.dtype == FA_DTYPE_BF16)
    kvcache_prep_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(c, q_follows_rows);
  else
    kvcache_prep_kernel<__half><<<grid, 128, 0, st>>>(c, q_follows_rows);
  return fa_host::check_launch("kvcache_prep_kernel");
}

}  // namespace fa
