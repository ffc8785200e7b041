// Merge of partial attention results by log-sum-exp.  Same math as combine_attn_seqk_parallel
// (csrc/flash_attn/src/flash_fwd_kernel.h:1169-1327): LSE = logsumexp_s(LSE_s),
// O = sum_s exp(LSE_s - LSE) * O_s; a row whose parts are all empty (-inf) gets O = 0, LSE = +inf.
#include "fa_common.cuh"

namespace fa {

struct CombineParams {
  const float* out_parts;  // (n_parts, rows, D)
  const float* lse_parts;  // (n_parts, rows)
  void* out;
  float* lse;  // may be NULL
  int64_t out_sb, out_ss, out_sh;
  int32_t n_parts, B, H, S, D, lse_pitch;
};

template <typename T>
__global__ void __launch_bounds__(128) combine_kernel(const CombineParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.B * p.H * p.S;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  // up to 128 parts: 4 per lane
  float l[4];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int s = lane + 32 * i;
    l[i] = s < p.n_parts ? p.lse_parts[(int64_t)s * rows + row] : -INFINITY;
    mx = fmaxf(mx, l[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  const float msafe = mx == -INFINITY ? 0.f : mx;
#pragma unroll
  for (int i = 0; i < 4; ++i) sum += __expf(l[i] - msafe);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const bool empty = !(sum > 0.f) || mx == -INFINITY;
  const float lse = empty ? INFINITY : logf(sum) + mx;
  const int s_idx = (int)(row % p.S);
  const int64_t bh = row / p.S;
  const int h = (int)(bh % p.H), b = (int)(bh / p.H);
  if (lane == 0 && p.lse) p.lse[bh * p.lse_pitch + s_idx] = lse;
  T* o = reinterpret_cast<T*>(p.out) + b * p.out_sb + s_idx * p.out_ss + h * p.out_sh;
  // head_dim <= 256: at most two 4-column groups per lane
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  float wgt[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) wgt[i] = empty ? 0.f : __expf(l[i] - lse);
  for (int s = 0; s < p.n_parts; ++s) {  // uniform trip count: every lane takes part in the shuffle
    float wsel = (s >> 5) == 0 ? wgt[0] : (s >> 5) == 1 ? wgt[1] : (s >> 5) == 2 ? wgt[2] : wgt[3];
    float w = __shfl_sync(0xffffffffu, wsel, s & 31);
    if (w == 0.f) continue;
    const float* src = p.out_parts + ((int64_t)s * rows + row) * p.D;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int c = lane * 4 + i * 128;
      if (c < p.D) {
        float4 x = *reinterpret_cast<const float4*>(src + c);
        acc[i].x += w * x.x;
        acc[i].y += w * x.y;
        acc[i].z += w * x.z;
        acc[i].w += w * x.w;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int c = lane * 4 + i * 128;
    if (c < p.D) {
      uint2 pk;
      pk.x = Pack<T>::two(acc[i].x, acc[i].y);
      pk.y = Pack<T>::two(acc[i].z, acc[i].w);
      *reinterpret_cast<uint2*>(o + c) = pk;
    }
  }
}

int combine(const float* out_parts, const float* lse_parts, const FaTensor& out, float* lse, int lse_pitch, int n_parts,
            int B, int H, int S, int D, int dtype, cudaStream_t st) {
  CombineParams p{out_parts, lse_parts, out.ptr, lse, out.stride_b, out.stride_s, out.stride_h, n_parts, B, H, S, D, lse_pitch};
  int64_t rows = (int64_t)B * H * S;
  unsigned grid = (unsigned)((rows + 3) / 4);
  if (dtype == FA_DTYPE_BF16)
    combine_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(p);
  else
    combine_kernel<__half><<<grid, 128, 0, st>>>(p);
  return fa_host::check_launch("combine_kernel");
}

// ---------------------------------------------------------------------------------------------
// In-place merge of one more partial result into a running fp32 accumulator (the per-step update of
// context-parallel ring attention): acc <- acc * exp(la - l) + part * exp(lb - l), la <- l, with
// l = logaddexp(la, lb).  An LSE of +inf (the kernels' "row saw no key") or -inf means empty.
struct MergeParams {
  float* acc;
  float* lse_acc;
  const void* part;
  const float* lse_part;
  int64_t acc_sb, acc_ss, acc_sh, part_sb, part_ss, part_sh;
  int64_t lacc_sb, lacc_sh, lpart_sb, lpart_sh;
  int32_t B, S, H, D;
};

template <typename T>
__global__ void __launch_bounds__(256) merge_partial_kernel(const MergeParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.B * p.S * p.H;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int h = (int)(row % p.H);
  const int s = (int)((row / p.H) % p.S);
  const int b = (int)(row / ((int64_t)p.H * p.S));
  float* la_p = p.lse_acc + b * p.lacc_sb + h * p.lacc_sh + s;
  float la = *la_p, lb = p.lse_part[b * p.lpart_sb + h * p.lpart_sh + s];
  if (la == INFINITY) la = -INFINITY;
  if (lb == INFINITY) lb = -INFINITY;
  const float mx = fmaxf(la, lb);
  float wa = 0.f, wb = 0.f, l = -INFINITY;
  if (mx != -INFINITY) {
    const float ea = __expf(la - mx), eb = __expf(lb - mx);
    const float inv = 1.f / (ea + eb);
    wa = ea * inv;
    wb = eb * inv;
    l = mx + __logf(ea + eb);
  }
  float* a = p.acc + b * p.acc_sb + s * p.acc_ss + h * p.acc_sh;
  const T* o = reinterpret_cast<const T*>(p.part) + b * p.part_sb + s * p.part_ss + h * p.part_sh;
  for (int c = lane * 4; c < p.D; c += 128) {
    float4 x = *reinterpret_cast<float4*>(a + c);
    const uint2 y = *reinterpret_cast<const uint2*>(o + c);
    x.x = wa * x.x + wb * Pack<T>::lo(y.x);
    x.y = wa * x.y + wb * Pack<T>::hi(y.x);
    x.z = wa * x.z + wb * Pack<T>::lo(y.y);
    x.w = wa * x.w + wb * Pack<T>::hi(y.y);
    *reinterpret_cast<float4*>(a + c) = x;
  }
  if (lane == 0) *la_p = l;
}

int merge_partial(const FaTensor& acc, float* lse_acc, int64_t lacc_sb, int64_t lacc_sh, const FaTensor& part,
                  const float* lse_part, int64_t lpart_sb, int64_t lpart_sh, int B, int S, int H, int D, int dtype,
                  cudaStream_t st) {
  MergeParams p{reinterpret_cast<float*>(acc.ptr), lse_acc, part.ptr, lse_part, acc.stride_b, acc.stride_s, acc.stride_h,
                part.stride_b, part.stride_s, part.stride_h, lacc_sb, lacc_sh, lpart_sb, lpart_sh, B, S, H, D};
  const int64_t rows = (int64_t)p.B * p.S * p.H;
  if (rows == 0) return 0;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == FA_DTYPE_BF16)
    merge_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
  else
    merge_partial_kernel<__half><<<grid, 256, 0, st>>>(p);
  return fa_host::check_launch("merge_partial_kernel");
}

}  // namespace fa
