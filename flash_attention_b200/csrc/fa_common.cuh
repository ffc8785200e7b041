// Shared device/host helpers of libfa_b200: sequence bookkeeping, the mask rule, dtype packing,
// legacy mma.sync / ldmatrix wrappers used by the any-shape kernels, and the dropout generator.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fa_b200.h"

namespace fa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Per-(batch) view of one attention problem.  Mirrors the role of BlockInfo
// (csrc/flash_attn/src/block_info.h:11-42): where the rows of this batch element start and how
// many there are, for fixed-length, packed (cu_seqlens) and KV-cache (seqused_k) inputs.
struct SeqInfo {
  int64_t q_row0;  // first row of this sequence in the packed q/out/dout/dq tensors (0 if batched)
  int64_t k_row0;
  int64_t q_batch;  // batch index to apply stride_b to (0 if packed)
  int64_t k_batch;
  int sq, sk;
  int shift;  // mask diagonal: key j visible iff i + shift - wl <= j <= i + shift + wr
};

__device__ __forceinline__ SeqInfo seq_info(const int32_t* cu_q, const int32_t* cu_k, const int32_t* seqused_k,
                                            const int32_t* kv_batch_idx, int seqlen_q, int seqlen_k, int use_shift,
                                            int mask_shift, int b, int seqused_extra = 0) {
  SeqInfo s;
  if (cu_q) {
    int q0 = cu_q[b];
    s.q_row0 = q0;
    s.sq = cu_q[b + 1] - q0;
    s.q_batch = 0;
  } else {
    s.q_row0 = 0;
    s.sq = seqlen_q;
    s.q_batch = b;
  }
  if (cu_k) {
    int k0 = cu_k[b];
    s.k_row0 = k0;
    s.sk = cu_k[b + 1] - k0;
    s.k_batch = 0;
  } else {
    s.k_row0 = 0;
    s.sk = seqused_k ? seqused_k[b] + seqused_extra : seqlen_k;
    s.k_batch = kv_batch_idx ? kv_batch_idx[b] : b;
  }
  s.shift = use_shift ? mask_shift : (s.sk - s.sq);
  return s;
}

// The mask rule of csrc/flash_attn/src/softmax.h:142-179 (bottom-right aligned causal / window).
__device__ __forceinline__ bool visible(int i, int j, int sk, int shift, int wl, int wr) {
  if (j >= sk) return false;
  if (wr >= 0 && j > i + shift + wr) return false;
  if (wl >= 0 && j < i + shift - wl) return false;
  return true;
}

// Range of key blocks [lo, hi) of width BN that rows [m0, m0+BM) can see.
__device__ __forceinline__ void key_block_range(int m0, int BM, int BN, int sk, int shift, int wl, int wr, int& lo,
                                                int& hi) {
  int nb = (sk + BN - 1) / BN;
  hi = nb;
  lo = 0;
  if (wr >= 0) {
    int jmax = m0 + BM - 1 + shift + wr;
    int h = jmax < 0 ? 0 : jmax / BN + 1;
    hi = h < nb ? h : nb;
  }
  if (wl >= 0) {
    int jmin = m0 + shift - wl;
    lo = jmin <= 0 ? 0 : jmin / BN;
  }
  if (hi < lo) hi = lo;
}

// Range of query blocks [lo, hi) of height BM that can see keys [n0, n0+BN).
__device__ __forceinline__ void query_block_range(int n0, int BN, int BM, int sq, int shift, int wl, int wr, int& lo,
                                                  int& hi) {
  int mb = (sq + BM - 1) / BM;
  lo = 0;
  hi = mb;
  if (wr >= 0) {
    int imin = n0 - shift - wr;
    lo = imin <= 0 ? 0 : imin / BM;
  }
  if (wl >= 0) {
    int imax = n0 + BN - 1 - shift + wl;
    int h = imax < 0 ? 0 : imax / BM + 1;
    hi = h < mb ? h : mb;
  }
  if (hi < lo) hi = lo;
}

template <typename T>
struct Pack;
template <>
struct Pack<__half> {
  static __device__ __forceinline__ uint32_t two(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float lo(uint32_t u) { return __low2float(*reinterpret_cast<__half2*>(&u)); }
  static __device__ __forceinline__ float hi(uint32_t u) { return __high2float(*reinterpret_cast<__half2*>(&u)); }
  static __device__ __forceinline__ float one(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from(float x) { return __float2half_rn(x); }
};
template <>
struct Pack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t two(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
  static __device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
  static __device__ __forceinline__ float one(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from(float x) { return __float2bfloat16_rn(x); }
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- legacy warp-level tensor-core path (any-shape kernels only) ----------------------------
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// ---- dropout -------------------------------------------------------------------------------
// Philox-4x32 with 7 rounds, the generator of csrc/flash_attn/src/philox.cuh:31-49.  One call
// yields 16 random bytes; an attention entry is KEPT iff its byte <= keep_threshold, where
// keep_threshold = floor(p_keep * 255) (flash_api.cpp:104, softmax.h:217-283).
__device__ __forceinline__ uint4 philox4x32_7(uint64_t seed, uint64_t subsequence, uint64_t offset) {
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  uint32_t c0 = (uint32_t)offset, c1 = (uint32_t)(offset >> 32), c2 = (uint32_t)subsequence,
           c3 = (uint32_t)(subsequence >> 32);
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0;
    c1 = n1;
    c2 = n2;
    c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// The random byte that decides entry (row, col) of head `bh`.  The entry belongs to the 16x32 tile
// (row/16, col/32); inside it, "lane" (row%8)*4 + (col%8)/2 draws one Philox block and the byte is
// picked by ((row%16)/8, (col%32)/8, col%2).  This is the reference's tiling (one Philox call per
// thread per 16x32 tile, softmax.h:233-237) stated as a pure function of (row, col), so that the
// forward, the backward and the returned mask agree whatever tile shapes the kernels use.
__device__ __forceinline__ uint4 dropout_block(uint64_t seed, uint64_t offset, int bh, int row16, int col32, int lane) {
  uint64_t subseq = ((uint64_t)(uint32_t)row16) | ((uint64_t)(uint32_t)col32 << 32);
  return philox4x32_7(seed, subseq, offset + (uint64_t)bh * 32 + lane);
}
__device__ __forceinline__ uint32_t dropout_byte_of(const uint4& blk, int r8, int nt, int e) {
  int idx = r8 * 8 + nt * 2 + e;  // 0..15
  uint32_t w = idx < 4 ? blk.x : idx < 8 ? blk.y : idx < 12 ? blk.z : blk.w;
  return (w >> ((idx & 3) * 8)) & 0xffu;
}
__device__ __forceinline__ uint32_t dropout_byte(uint64_t seed, uint64_t offset, int bh, int row, int col) {
  uint4 blk = dropout_block(seed, offset, bh, row >> 4, col >> 5, (row & 7) * 4 + ((col & 7) >> 1));
  return dropout_byte_of(blk, (row & 15) >> 3, (col & 31) >> 3, col & 1);
}

}  // namespace fa

// ---- host side ------------------------------------------------------------------------------
namespace fa_host {
void set_error(const char* fmt, ...);
int check_launch(const char* what);
int sm_count();

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to one device: a kernel's launcher keeps
// one of these (a static, zero-initialised) and raises the limit once per device, not once per process.
struct DeviceOnce {
  bool done[64];
};
// true when the caller still has to do its per-device set-up for `dev` (and marks it done); devices
// outside the table are never marked, so their set-up simply runs on every call.
inline bool device_once_needed(DeviceOnce& once, int dev) {
  if (dev < 0 || dev >= 64) return true;
  if (once.done[dev]) return false;
  once.done[dev] = true;
  return true;
}
int raise_smem_limit(DeviceOnce& once, const void* kernel, int bytes, const char* name);
}  // namespace fa_host

#define FA_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      fa_host::set_error(__VA_ARGS__);   \
      return 1;                          \
    }                                    \
  } while (0)
