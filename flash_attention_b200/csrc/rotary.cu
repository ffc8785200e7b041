// Rotary position embedding applied to (batch, seqlen, heads, head_dim) or packed (total, heads,
// head_dim) 16-bit tensors, the step right before attention in the reference's MHA module.
// Same semantics as rotary_kernel / apply_rotary (flash_attn/ops/triton/rotary.py:17-140, 143-240):
//   the first rotary_dim elements of every row are rotated by the angle of position
//   s + seqlen_offset[b] (cos = 1, sin = 0 past the end of the tables), either as halves
//   (x0 = x[:r/2], x1 = x[r/2:r]) or as interleaved pairs (x[2i], x[2i+1]):
//     o0 = x0 cos - x1 sin,  o1 = x0 sin + x1 cos     (sin negated for the conjugate = backward),
//   computed in fp32; elements past rotary_dim are copied when out != x.
// Pure streaming work: one thread per 16-byte piece of a row (plus its partner piece in the
// second half), consecutive threads on consecutive pieces, rows in memory order.
#include "fa_common.cuh"

namespace fa {

struct RotaryParams {
  FaRotaryArgs a;
  int n_rot;   // 16-byte pieces per row that rotate
  int n_tail;  // 16-byte pieces per row that are only copied
};

__device__ __forceinline__ int rotary_position(const FaRotaryArgs& a, int64_t tok, int& b, int& s) {
  // returns the table row of token `tok` (row index over batch x seqlen, or over the packed total)
  if (a.cu_seqlens) {
    int lo = 0, hi = a.batch;  // largest b with cu_seqlens[b] <= tok
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.cu_seqlens[mid] <= tok) lo = mid; else hi = mid;
    }
    b = lo;
    s = (int)(tok - a.cu_seqlens[lo]);
  } else {
    b = (int)(tok / a.seqlen);
    s = (int)(tok - (int64_t)b * a.seqlen);
  }
  return s + (a.seqlen_offsets ? a.seqlen_offsets[b] : a.seqlen_offset);
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  f[0] = Pack<T>::lo(v.x); f[1] = Pack<T>::hi(v.x); f[2] = Pack<T>::lo(v.y); f[3] = Pack<T>::hi(v.y);
  f[4] = Pack<T>::lo(v.z); f[5] = Pack<T>::hi(v.z); f[6] = Pack<T>::lo(v.w); f[7] = Pack<T>::hi(v.w);
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  uint4 v;
  v.x = Pack<T>::two(f[0], f[1]); v.y = Pack<T>::two(f[2], f[3]);
  v.z = Pack<T>::two(f[4], f[5]); v.w = Pack<T>::two(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

// Vector form: rotary_dim / 2 (halves) or rotary_dim (interleaved) and head_dim are multiples of 8
// and every row starts on a 16-byte boundary.
template <typename T, bool kInterleaved>
__global__ void __launch_bounds__(256) rotary_vec_kernel(const __grid_constant__ RotaryParams p) {
  const FaRotaryArgs& a = p.a;
  const int per_row = p.n_rot + p.n_tail;
  const int64_t rows = (a.cu_seqlens ? (int64_t)a.total : (int64_t)a.batch * a.seqlen) * a.heads;
  const int64_t items = rows * per_row;
  for (int64_t it = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = it / per_row;
    const int c = (int)(it - row * per_row);
    const int64_t tok = row / a.heads;
    const int h = (int)(row - tok * a.heads);
    int b, s;
    const int pos = rotary_position(a, tok, b, s);
    const int64_t srow = a.cu_seqlens ? tok : (int64_t)s;  // packed tensors have no batch stride
    const int64_t bsel = a.cu_seqlens ? 0 : b;
    const T* x = reinterpret_cast<const T*>(a.x.ptr) + bsel * a.x.stride_b + srow * a.x.stride_s + (int64_t)h * a.x.stride_h;
    T* o = reinterpret_cast<T*>(a.out.ptr) + bsel * a.out.stride_b + srow * a.out.stride_s + (int64_t)h * a.out.stride_h;
    if (c >= p.n_rot) {  // copy-only tail
      const int e = a.rotary_dim + (c - p.n_rot) * 8;
      *reinterpret_cast<uint4*>(o + e) = *reinterpret_cast<const uint4*>(x + e);
      continue;
    }
    const int half = a.rotary_dim >> 1;
    const bool in_table = pos >= 0 && pos < a.seqlen_ro;
    const T* cs = reinterpret_cast<const T*>(a.cos) + (int64_t)pos * half;
    const T* sn = reinterpret_cast<const T*>(a.sin) + (int64_t)pos * half;
    if (!kInterleaved) {
      float x0[8], x1[8], cf[8], sf[8], o0[8], o1[8];
      load8(x + c * 8, x0);
      load8(x + half + c * 8, x1);
      if (in_table) {
        load8(cs + c * 8, cf);
        load8(sn + c * 8, sf);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) { cf[i] = 1.f; sf[i] = 0.f; }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float sv = a.conjugate ? -sf[i] : sf[i];
        o0[i] = x0[i] * cf[i] - x1[i] * sv;
        o1[i] = x0[i] * sv + x1[i] * cf[i];
      }
      store8(o + c * 8, o0);
      store8(o + half + c * 8, o1);
    } else {
      float xv[8], ov[8], cf[4], sf[4];
      load8(x + c * 8, xv);
      if (in_table) {
        const uint2 cv = *reinterpret_cast<const uint2*>(cs + c * 4), sv = *reinterpret_cast<const uint2*>(sn + c * 4);
        cf[0] = Pack<T>::lo(cv.x); cf[1] = Pack<T>::hi(cv.x); cf[2] = Pack<T>::lo(cv.y); cf[3] = Pack<T>::hi(cv.y);
        sf[0] = Pack<T>::lo(sv.x); sf[1] = Pack<T>::hi(sv.x); sf[2] = Pack<T>::lo(sv.y); sf[3] = Pack<T>::hi(sv.y);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) { cf[i] = 1.f; sf[i] = 0.f; }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float sv = a.conjugate ? -sf[i] : sf[i];
        ov[2 * i] = xv[2 * i] * cf[i] - xv[2 * i + 1] * sv;
        ov[2 * i + 1] = xv[2 * i] * sv + xv[2 * i + 1] * cf[i];
      }
      store8(o + c * 8, ov);
    }
  }
}

// Any rotary_dim / alignment: one thread per rotated pair, then per copied element.
template <typename T>
__global__ void __launch_bounds__(256) rotary_scalar_kernel(const __grid_constant__ RotaryParams p) {
  const FaRotaryArgs& a = p.a;
  const int half = a.rotary_dim >> 1;
  const int tail = a.out.ptr != a.x.ptr ? a.head_dim - a.rotary_dim : 0;
  const int per_row = half + tail;
  const int64_t rows = (a.cu_seqlens ? (int64_t)a.total : (int64_t)a.batch * a.seqlen) * a.heads;
  const int64_t items = rows * per_row;
  for (int64_t it = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = it / per_row;
    const int c = (int)(it - row * per_row);
    const int64_t tok = row / a.heads;
    const int h = (int)(row - tok * a.heads);
    int b, s;
    const int pos = rotary_position(a, tok, b, s);
    const int64_t srow = a.cu_seqlens ? tok : (int64_t)s;
    const int64_t bsel = a.cu_seqlens ? 0 : b;
    const T* x = reinterpret_cast<const T*>(a.x.ptr) + bsel * a.x.stride_b + srow * a.x.stride_s + (int64_t)h * a.x.stride_h;
    T* o = reinterpret_cast<T*>(a.out.ptr) + bsel * a.out.stride_b + srow * a.out.stride_s + (int64_t)h * a.out.stride_h;
    if (c >= half) {
      const int e = a.rotary_dim + (c - half);
      o[e] = x[e];
      continue;
    }
    float cv = 1.f, sv = 0.f;
    if (pos >= 0 && pos < a.seqlen_ro) {
      cv = Pack<T>::one(reinterpret_cast<const T*>(a.cos)[(int64_t)pos * half + c]);
      sv = Pack<T>::one(reinterpret_cast<const T*>(a.sin)[(int64_t)pos * half + c]);
    }
    if (a.conjugate) sv = -sv;
    const int i0 = a.interleaved ? 2 * c : c, i1 = a.interleaved ? 2 * c + 1 : c + half;
    const float x0 = Pack<T>::one(x[i0]), x1 = Pack<T>::one(x[i1]);
    o[i0] = Pack<T>::from(x0 * cv - x1 * sv);
    o[i1] = Pack<T>::from(x0 * sv + x1 * cv);
  }
}

template <typename T>
static int rotary_t(const FaRotaryArgs& a, cudaStream_t st) {
  RotaryParams p;
  p.a = a;
  const int64_t rows = (a.cu_seqlens ? (int64_t)a.total : (int64_t)a.batch * a.seqlen) * a.heads;
  if (rows == 0 || a.head_dim == 0) return 0;
  const int half = a.rotary_dim / 2;
  const bool inplace = a.out.ptr == a.x.ptr;
  auto aligned = [](const FaTensor& t) {
    return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && t.stride_b % 8 == 0 && t.stride_s % 8 == 0 && t.stride_h % 8 == 0;
  };
  const int unit = a.interleaved ? a.rotary_dim : half;
  const bool vec = aligned(a.x) && aligned(a.out) && unit % 8 == 0 && a.head_dim % 8 == 0 && a.rotary_dim % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(a.cos) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.sin) & 15) == 0 && half % 8 == 0;
  const int sms = fa_host::sm_count();
  if (vec) {
    p.n_rot = unit / 8;
    p.n_tail = inplace ? 0 : (a.head_dim - a.rotary_dim) / 8;
    const int64_t items = rows * (p.n_rot + p.n_tail);
    if (items == 0) return 0;
    const int64_t want = (items + 255) / 256;
    const unsigned grid = (unsigned)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);  // one resident wave, grid-stride
    if (a.interleaved)
      rotary_vec_kernel<T, true><<<grid, 256, 0, st>>>(p);
    else
      rotary_vec_kernel<T, false><<<grid, 256, 0, st>>>(p);
    return fa_host::check_launch("rotary_vec_kernel");
  }
  p.n_rot = p.n_tail = 0;
  const int64_t items = rows * (half + (inplace ? 0 : a.head_dim - a.rotary_dim));
  if (items == 0) return 0;
  const int64_t want = (items + 255) / 256;
  const unsigned grid = (unsigned)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);  // one resident wave, grid-stride
  rotary_scalar_kernel<T><<<grid, 256, 0, st>>>(p);
  return fa_host::check_launch("rotary_scalar_kernel");
}

int rotary(const FaRotaryArgs& a, cudaStream_t st) {
  return a.dtype == FA_DTYPE_BF16 ? rotary_t<__nv_bfloat16>(a, st) : rotary_t<__half>(a, st);
}

}  // namespace fa
