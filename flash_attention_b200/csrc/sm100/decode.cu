// Fused single-step decode against a KV cache: split-KV streaming attention with in-kernel
// append of the new token (rotary on K and Q).  HBM-bandwidth bound by construction: every K and
// V row that is attended to is read exactly once, by TMA, into a ring of shared-memory slots.
//
// Replaces compute_attn_1rowblock_splitkv (csrc/flash_attn/src/flash_fwd_kernel.h:584-1130) for
// the decode shape: few query rows per KV head (seqlen_q x heads/heads_k <= 16), no mask window.
// The combine step is shared with the other split paths (combine.cu).
//
// Grid (num_splits, heads_k, batch).  A CTA owns the keys [split*chunk, (split+1)*chunk) of one
// (batch, KV head) and ALL query rows that share that KV head (the grouped-query trick of
// flash_api.cpp:1096-1104: the cache is read once per KV head, not once per query head).
// Warps: 0-3 consumers (each takes 16 of the 64 keys of a tile with its own online-softmax state,
// merged at the end), warp 4 = TMA producer.  Q.K^T and P.V use warp-level mma.sync m16n8k16 —
// 4 useful rows of 16, irrelevant next to the memory time — fed by ldmatrix from the 128B-swizzled
// tiles that TMA wrote.
// Paged cache (block_table): the same two tensor maps then describe (page, row in page, head, dim), and the
// producer looks the page of each 64-key tile up in the table; nothing else changes.
// New token: the CTA whose key range contains position L = cache_seqlens[b] rotates k_new at L,
// writes it and v_new to the cache in global memory AND patches them into its shared-memory tile,
// so no CTA reads a row of global memory that this launch writes.
#include "../fa_common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace fa {

using namespace ptx;

StatusRef status_ref(bool may_allocate);

namespace {

constexpr int kTileKeys = 64;
constexpr int kStages = 3;
constexpr int kMaxRows = 16;
constexpr int kChunkKeys = 2048;  // target keys per split

enum DecWait { W_DEC_FULL = 31, W_DEC_EMPTY = 32 };

struct DecodeParams {
  CUtensorMap tk, tv;
  FaKvcacheArgs a;
  int num_splits;
  int keys_per_split;  // multiple of kTileKeys
  StatusRef status;
};

template <int D>
struct DCfg {
  static constexpr int BOX_BYTES = kTileKeys * 128;       // 64 keys x 64 elements x 2 B
  static constexpr int NBOX = D / 64;
  static constexpr int TILE_BYTES = NBOX * BOX_BYTES;     // one K or V tile
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int Q_LD = D + 8;
  static constexpr int Q_BYTES = kMaxRows * Q_LD * 2;
  static constexpr int SMEM_BYTES = kStages * STAGE_BYTES + Q_BYTES + (2 * kStages + 1) * 8 + 32 + 1024;
};

// address of (row, 16-byte chunk c16 of the 128-byte row) inside one swizzled TMA box
__device__ __forceinline__ uint32_t swz(uint32_t box_base, int row, int c16) {
  return box_base + row * 128 + (((c16 ^ row) & 7) << 4);
}

template <typename T>
__device__ __forceinline__ void rotate8(float (&x)[8], const float (&xp)[8], const T* cosr, const T* sinr, int d0,
                                        int rdim, bool interleaved) {
  // x holds dims d0..d0+7 (d0 % 8 == 0); xp the partner values for the non-interleaved pairing.
  if (d0 >= rdim) return;
  const int half = rdim >> 1;
  if (interleaved) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const int idx = (d0 + i) >> 1;
      const float c = Pack<T>::one(cosr[idx]), s = Pack<T>::one(sinr[idx]);
      const float a = x[i], b2 = x[i + 1];
      x[i] = a * c - b2 * s;
      x[i + 1] = a * s + b2 * c;
    }
  } else {
    const bool first = d0 < half;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = first ? d0 + i : d0 + i - half;
      const float c = Pack<T>::one(cosr[idx]), s = Pack<T>::one(sinr[idx]);
      x[i] = first ? x[i] * c - xp[i] * s : x[i] * c + xp[i] * s;
    }
  }
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  x[0] = Pack<T>::lo(u.x);
  x[1] = Pack<T>::hi(u.x);
  x[2] = Pack<T>::lo(u.y);
  x[3] = Pack<T>::hi(u.y);
  x[4] = Pack<T>::lo(u.z);
  x[5] = Pack<T>::hi(u.z);
  x[6] = Pack<T>::lo(u.w);
  x[7] = Pack<T>::hi(u.w);
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  uint4 u;
  u.x = Pack<T>::two(x[0], x[1]);
  u.y = Pack<T>::two(x[2], x[3]);
  u.z = Pack<T>::two(x[4], x[5]);
  u.w = Pack<T>::two(x[6], x[7]);
  return u;
}

// Rotated copy of 8 dims [d0, d0+8) of a row (rotary at table row cosr/sinr, or plain when null).
template <typename T>
__device__ __forceinline__ uint4 rotated_chunk(const T* row, int d0, const T* cosr, const T* sinr, int rdim,
                                               bool interleaved) {
  float x[8], xp[8];
  load8<T>(row + d0, x);
  if (cosr != nullptr && d0 < rdim) {
    if (!interleaved) {
      const int half = rdim >> 1;
      load8<T>(row + (d0 < half ? d0 + half : d0 - half), xp);
    }
    rotate8<T>(x, xp, cosr, sinr, d0, rdim, interleaved);
  }
  return pack8<T>(x);
}

template <typename T, int D>
__global__ void __launch_bounds__(160, 2) decode_kernel(const __grid_constant__ DecodeParams P) {
  using C = DCfg<D>;
  const FaKvcacheArgs& a = P.a;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_addr(smem);
  T* sQ = reinterpret_cast<T*>(smem + kStages * C::STAGE_BYTES);
  const uint32_t bar0 = s_base + kStages * C::STAGE_BYTES + C::Q_BYTES;
  auto bar_full = [&](int s) { return bar0 + 8 * s; };
  auto bar_empty = [&](int s) { return bar0 + 8 * (kStages + s); };
  const uint32_t bar_rdv = bar0 + 8 * 2 * kStages;  // rendezvous of the four consumer warps
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kStages * C::STAGE_BYTES + C::Q_BYTES + (2 * kStages + 1) * 8 + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = a.heads / a.heads_k;
  const int M = a.seqlen_q * group;  // query rows that share this KV head (<= 16)
  const int L = a.cache_seqlens ? a.cache_seqlens[b] : a.seqlen_cache;
  const bool has_new = a.knew.ptr != nullptr;
  const int Ltot = min(L + (has_new ? 1 : 0), a.seqlen_cache);
  const int cb = a.cache_batch_idx ? a.cache_batch_idx[b] : b;
  // paged cache: the tensor maps describe (page, row in page); a 64-key tile never straddles a page
  const int32_t* pages = a.block_table ? a.block_table + (int64_t)b * a.block_table_stride : nullptr;
  const int key_lo = split * P.keys_per_split;
  const int key_hi = min(key_lo + P.keys_per_split, Ltot);
  const int nsplit = P.num_splits;
  const int64_t rows_total = (int64_t)a.batch * a.heads * a.seqlen_q;

  auto row_index = [&](int r) {  // flat (batch, head, seq) index of query row r of this KV head
    const int s = r / group, gi = r % group;
    return ((int64_t)b * a.heads + (hk * group + gi)) * a.seqlen_q + s;
  };

  if (key_hi <= key_lo) {
    // nothing to attend in this split: an empty part (LSE = -inf), or zeros if it is the only part
    if (tid < M) {
      const int64_t ri = row_index(tid);
      if (nsplit > 1) {
        a.lse_accum[(int64_t)split * rows_total + ri] = -INFINITY;
      } else {
        a.softmax_lse[ri] = INFINITY;
        const int s = tid / group, gi = tid % group;
        T* o = reinterpret_cast<T*>(a.out.ptr) + b * a.out.stride_b + s * a.out.stride_s + (hk * group + gi) * a.out.stride_h;
        for (int d = 0; d < D; d += 8) *reinterpret_cast<uint4*>(o + d) = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  const int ntiles = (key_hi - key_lo + kTileKeys - 1) / kTileKeys;

  if (tid == 0) {
    abort_init(abort_flag, P.status);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 4);
    }
    mbar_init(bar_rdv, 4);
    fence_barrier_init();
    fence_proxy_async();
  }
  // stage Q (rotated at position L) as [16][D+8], zero rows beyond M
  const T* cosr = a.rotary_cos ? reinterpret_cast<const T*>(a.rotary_cos) + (int64_t)L * (a.rotary_dim / 2) : nullptr;
  const T* sinr = a.rotary_sin ? reinterpret_cast<const T*>(a.rotary_sin) + (int64_t)L * (a.rotary_dim / 2) : nullptr;
  if (L >= a.seqlen_ro) cosr = sinr = nullptr;
  for (int i = tid; i < kMaxRows * (D / 8); i += blockDim.x) {
    const int r = i / (D / 8), d0 = (i % (D / 8)) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (r < M) {
      const int s = r / group, gi = r % group;
      const T* qrow = reinterpret_cast<const T*>(a.q.ptr) + b * a.q.stride_b + s * a.q.stride_s + (hk * group + gi) * a.q.stride_h;
      val = rotated_chunk<T>(qrow, d0, cosr, sinr, a.rotary_dim, a.rotary_interleaved != 0);
    }
    *reinterpret_cast<uint4*>(sQ + r * C::Q_LD + d0) = val;
  }
  __syncthreads();

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&P.tk);
      prefetch_tensormap(&P.tv);
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int slot = i % kStages, round = i / kStages;
        ok = mbar_wait(bar_empty(slot), (round & 1) ^ 1, W_DEC_EMPTY, abort_flag);
        if (!ok) break;
        const uint32_t dst = s_base + slot * C::STAGE_BYTES;
        mbar_expect_tx(bar_full(slot), C::STAGE_BYTES);
        const int key0 = key_lo + i * kTileKeys;
        const int row0 = pages ? key0 % a.page_block_size : key0;
        const int slab = pages ? pages[key0 / a.page_block_size] : cb;
        for (int c = 0; c < C::NBOX; ++c) tma_load_4d(dst + c * C::BOX_BYTES, &P.tk, bar_full(slot), c * 64, row0, hk, slab);
        for (int c = 0; c < C::NBOX; ++c)
          tma_load_4d(dst + C::TILE_BYTES + c * C::BOX_BYTES, &P.tv, bar_full(slot), c * 64, row0, hk, slab);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers (warps 0-3)
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    ldsm_x4(qf[ks], smem_u32(sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::Q_LD + ks * 16 + (lane >> 4) * 8));
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float scale_log2 = a.softmax_scale * kLog2e;
  bool ok = true;
  int rdv_phase = 0;
  // bounded rendezvous of the consumer warps (instead of bar.sync, which could strand a warp if
  // another one has given up on a wait)
  auto rendezvous = [&]() {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_rdv);
    const bool r = mbar_wait(bar_rdv, rdv_phase & 1, W_DEC_FULL, abort_flag);
    ++rdv_phase;
    return r;
  };

  for (int i = 0; i < ntiles; ++i) {
    const int slot = i % kStages;
    ok = mbar_wait(bar_full(slot), (i / kStages) & 1, W_DEC_FULL, abort_flag);
    if (!ok) break;
    const uint32_t sK = s_base + slot * C::STAGE_BYTES, sV = sK + C::TILE_BYTES;
    const int key0 = key_lo + i * kTileKeys;
    const bool tail = key0 + kTileKeys > Ltot;
    const bool holds_new = has_new && L >= key0 && L < key0 + kTileKeys && L < a.seqlen_cache;
    if (tail || holds_new) {
      // patch the tile: new K (rotated) / V row at position L, zero V rows that are past the end
      unsigned char* tileV = smem + slot * C::STAGE_BYTES + C::TILE_BYTES;
      unsigned char* tileK = smem + slot * C::STAGE_BYTES;
      if (holds_new) {
        const int r = L - key0;
        const T* kn = reinterpret_cast<const T*>(a.knew.ptr) + b * a.knew.stride_b + hk * a.knew.stride_h;
        const T* vn = reinterpret_cast<const T*>(a.vnew.ptr) + b * a.vnew.stride_b + hk * a.vnew.stride_h;
        const int64_t slab = pages ? pages[L / a.page_block_size] : cb;
        const int64_t srow = pages ? L % a.page_block_size : L;
        T* kg = reinterpret_cast<T*>(a.kcache.ptr) + slab * a.kcache.stride_b + srow * a.kcache.stride_s + hk * a.kcache.stride_h;
        T* vg = reinterpret_cast<T*>(a.vcache.ptr) + slab * a.vcache.stride_b + srow * a.vcache.stride_s + hk * a.vcache.stride_h;
        for (int c = tid; c < 2 * (D / 8); c += 128) {
          const bool is_v = c >= D / 8;
          const int d0 = (is_v ? c - D / 8 : c) * 8;
          uint4 val = is_v ? *reinterpret_cast<const uint4*>(vn + d0)
                           : rotated_chunk<T>(kn, d0, cosr, sinr, a.rotary_dim, a.rotary_interleaved != 0);
          *reinterpret_cast<uint4*>((is_v ? vg : kg) + d0) = val;
          unsigned char* box = (is_v ? tileV : tileK) + (d0 / 64) * C::BOX_BYTES;
          *reinterpret_cast<uint4*>(box + r * 128 + ((((d0 % 64) / 8) ^ r) & 7) * 16) = val;
        }
      }
      if (tail) {
        const int r_first = Ltot - key0;  // rows [r_first, 64) are past the end
        for (int c = tid; c < (kTileKeys - r_first) * (D / 8); c += 128) {
          const int r = r_first + c / (D / 8), d0 = (c % (D / 8)) * 8;
          unsigned char* box = tileV + (d0 / 64) * C::BOX_BYTES;
          *reinterpret_cast<uint4*>(box + r * 128 + ((((d0 % 64) / 8) ^ r) & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      fence_proxy_async();
      ok = rendezvous();
      if (!ok) break;
    }

    // S (16 rows x this warp's 16 keys)
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const int krow = warp * 16 + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t bb[4];
      const int c16 = (ks * 2 + ((lane >> 3) & 1)) & 7;
      ldsm_x4(bb, swz(sK + (ks / 4) * C::BOX_BYTES, krow, c16));
      mma16816<T>(s[0], qf[ks], bb[0], bb[1]);
      mma16816<T>(s[1], qf[ks], bb[2], bb[3]);
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + warp * 16 + nt * 8 + 2 * t + (e & 1);
        const float x = key < Ltot ? s[nt][e] * scale_log2 : -INFINITY;
        s[nt][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    float msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mn = fmaxf(m_run[r], mx[r]);
      msafe[r] = mn == -INFINITY ? 0.f : mn;
      const float alpha = fast_exp2(m_run[r] - msafe[r]);
      m_run[r] = mn;
      l_run[r] *= alpha;
#pragma unroll
      for (int i2 = 0; i2 < D / 8; ++i2) {
        o_acc[i2][2 * r] *= alpha;
        o_acc[i2][2 * r + 1] *= alpha;
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = fast_exp2(s[nt][e] - msafe[e >> 1]);
        l_run[e >> 1] += pv;
        s[nt][e] = pv;
      }
    uint32_t pa[4];
    pa[0] = Pack<T>::two(s[0][0], s[0][1]);
    pa[1] = Pack<T>::two(s[0][2], s[0][3]);
    pa[2] = Pack<T>::two(s[1][0], s[1][1]);
    pa[3] = Pack<T>::two(s[1][2], s[1][3]);
    const int vrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
      uint32_t bb[4];
      const int c16 = (dt * 2 + (lane >> 4)) & 7;
      ldsm_x4_t(bb, swz(sV + (dt / 4) * C::BOX_BYTES, vrow, c16));
      mma16816<T>(o_acc[2 * dt], pa, bb[0], bb[1]);
      mma16816<T>(o_acc[2 * dt + 1], pa, bb[2], bb[3]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty(slot));
  }

  // ---- merge the four warps, write the (partial) result
  if (ok) ok = rendezvous();  // all tiles consumed; the ring is free (no copy is in flight)
  if (!ok) return;
  float* sO = reinterpret_cast<float*>(smem);                 // [4 warps][16 rows][D]
  float* sM = reinterpret_cast<float*>(sQ);                    // [4][16] max, then [4][16] sum
  float* sL = sM + 64;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t == 0) {
      sM[warp * 16 + g + r * 8] = m_run[r];
      sL[warp * 16 + g + r * 8] = l;
    }
#pragma unroll
    for (int i2 = 0; i2 < D / 8; ++i2)
      *reinterpret_cast<float2*>(sO + (warp * 16 + g + r * 8) * D + i2 * 8 + 2 * t) = make_float2(o_acc[i2][2 * r], o_acc[i2][2 * r + 1]);
  }
  ok = rendezvous();
  if (ok) {
    // thread -> (row, 4 consecutive dims); D/4 threads per row
    for (int i = tid; i < M * (D / 4); i += 128) {
      const int r = i / (D / 4), d0 = (i % (D / 4)) * 4;
      float mw[4], mmax = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mw[w] = sM[w * 16 + r];
        mmax = fmaxf(mmax, mw[w]);
      }
      const float msafe = mmax == -INFINITY ? 0.f : mmax;
      float lsum = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = fast_exp2(mw[w] - msafe);
        lsum += f * sL[w * 16 + r];
        const float4 x = *reinterpret_cast<const float4*>(sO + (w * 16 + r) * D + d0);
        acc.x += f * x.x;
        acc.y += f * x.y;
        acc.z += f * x.z;
        acc.w += f * x.w;
      }
      const bool empty = !(lsum > 0.f);
      const float inv = empty ? 0.f : 1.f / lsum;
      const float lse = empty ? INFINITY : (mmax + log2f(lsum)) * kLn2;
      const int64_t ri = row_index(r);
      if (nsplit > 1) {
        *reinterpret_cast<float4*>(a.out_accum + ((int64_t)split * rows_total + ri) * D + d0) =
            make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        if (d0 == 0) a.lse_accum[(int64_t)split * rows_total + ri] = empty ? -INFINITY : lse;
      } else {
        const int s = r / group, gi = r % group;
        T* o = reinterpret_cast<T*>(a.out.ptr) + b * a.out.stride_b + s * a.out.stride_s + (hk * group + gi) * a.out.stride_h;
        uint2 pk;
        pk.x = Pack<T>::two(acc.x * inv, acc.y * inv);
        pk.y = Pack<T>::two(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(o + d0) = pk;
        if (d0 == 0) a.softmax_lse[ri] = lse;
      }
    }
  }
}

template <typename T, int D>
int launch_decode(const FaKvcacheArgs& a, int num_splits, int keys_per_split, cudaStream_t st, bool may_allocate) {
  using C = DCfg<D>;
  DecodeParams P;
  P.a = a;
  P.num_splits = num_splits;
  P.keys_per_split = keys_per_split;
  const int slab_rows = a.block_table ? a.page_block_size : a.seqlen_cache;  // rows of one page / of one sequence's cache
  if (make_tmap_4d(&P.tk, a.kcache, a.dtype, slab_rows, a.heads_k, a.batch_cache, a.head_dim, kTileKeys)) return 1;
  if (make_tmap_4d(&P.tv, a.vcache, a.dtype, slab_rows, a.heads_k, a.batch_cache, a.head_dim, kTileKeys)) return 1;
  auto kern = decode_kernel<T, D>;
  P.status = status_ref(may_allocate);
  static fa_host::DeviceOnce once;
  if (int rc = fa_host::raise_smem_limit(once, reinterpret_cast<const void*>(kern), C::SMEM_BYTES, "decode_kernel")) return rc;
  dim3 grid(num_splits, a.heads_k, a.batch);
  kern<<<grid, 160, C::SMEM_BYTES, st>>>(P);
  return fa_host::check_launch("decode_kernel");
}

int keys_per_split_of(const FaKvcacheArgs& a, int num_splits) {
  const int tiles = (a.seqlen_cache + kTileKeys - 1) / kTileKeys;
  return ((tiles + num_splits - 1) / num_splits) * kTileKeys;
}

}  // namespace

int combine(const float* out_parts, const float* lse_parts, const FaTensor& out, float* lse, int lse_pitch, int n_parts,
            int B, int H, int S, int D, int dtype, cudaStream_t st);

bool decode_eligible(const FaKvcacheArgs& a) {
  if (a.head_dim != 64 && a.head_dim != 128) return false;
  if (a.window_left >= 0 || a.window_right >= 0) return false;
  const int group = a.heads / a.heads_k;
  if (a.seqlen_q * group > kMaxRows || a.seqlen_q < 1) return false;
  if (a.knew.ptr && a.seqlen_new != 1) return false;
  if (a.rotary_cos && (a.rotary_dim % 16 != 0 || a.rotary_dim > a.head_dim)) return false;
  if (!tma_compatible(a.kcache) || !tma_compatible(a.vcache)) return false;
  if (a.seqlen_cache <= 0) return false;
  return encode_tiled_fn() != nullptr;
}

int decode_plan(const FaKvcacheArgs& a, int num_sms) {
  const int tiles = (a.seqlen_cache + kTileKeys - 1) / kTileKeys;
  int splits;
  if (a.num_splits >= 1) {
    splits = a.num_splits;
  } else {
    // enough CTAs to fill the machine twice, and no CTA longer than kChunkKeys keys so that
    // sequences of very different lengths still balance
    const int units = a.batch * a.heads_k;
    const int fill = (2 * num_sms + units - 1) / units;
    const int by_len = (a.seqlen_cache + kChunkKeys - 1) / kChunkKeys;
    splits = fill > by_len ? fill : by_len;
  }
  if (splits > 128) splits = 128;
  if (splits > tiles) splits = tiles;
  if (splits < 1) splits = 1;
  // drop splits that would be empty after rounding the chunk to whole tiles
  const int per = (tiles + splits - 1) / splits;
  splits = (tiles + per - 1) / per;
  return splits;
}

int decode_run(const FaKvcacheArgs& a, int num_splits, cudaStream_t st, bool may_allocate) {
  const int kps = keys_per_split_of(a, num_splits);
  const bool bf = a.dtype == FA_DTYPE_BF16;
  int rc;
  if (a.head_dim == 64)
    rc = bf ? launch_decode<__nv_bfloat16, 64>(a, num_splits, kps, st, may_allocate) : launch_decode<__half, 64>(a, num_splits, kps, st, may_allocate);
  else
    rc = bf ? launch_decode<__nv_bfloat16, 128>(a, num_splits, kps, st, may_allocate) : launch_decode<__half, 128>(a, num_splits, kps, st, may_allocate);
  if (rc) return rc;
  if (num_splits > 1)
    return combine(a.out_accum, a.lse_accum, a.out, a.softmax_lse, a.seqlen_q, num_splits, a.batch, a.heads, a.seqlen_q,
                   a.head_dim, a.dtype, st);
  return 0;
}

// ---- split-KV decode without any allocation by caller or library -------------------------------
// Scratch for the per-split partial results lives in this translation unit's device image: every
// GPU that loads the library reserves kNoAllocScratchBytes until the process exits.
constexpr size_t kNoAllocScratchBytes = 24u << 20;  // 24 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

size_t decode_noalloc_capacity() { return kNoAllocScratchBytes; }

static size_t noalloc_bytes_needed(const FaKvcacheArgs& a, int num_splits) {
  const size_t rows = (size_t)a.batch * a.heads * a.seqlen_q;
  const size_t lse_bytes = (rows * num_splits * sizeof(float) + 255) & ~size_t(255);
  return lse_bytes + rows * num_splits * (size_t)a.head_dim * sizeof(float);
}

// Largest split count <= `num_splits` (in the rounding of decode_plan) whose partials fit the
// built-in buffer; 1 always fits (a single split writes no partials).
int decode_noalloc_fit(const FaKvcacheArgs& a, int num_splits) {
  const int tiles = (a.seqlen_cache + kTileKeys - 1) / kTileKeys;
  while (num_splits > 1 && noalloc_bytes_needed(a, num_splits) > kNoAllocScratchBytes) {
    --num_splits;
    const int per = (tiles + num_splits - 1) / num_splits;
    num_splits = (tiles + per - 1) / per;
  }
  return num_splits;
}

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address; the
// address on the current device is looked up once per device and cached.
static int noalloc_scratch_ptr(unsigned char** out) {
  static unsigned char* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    fa_host::set_error("fa_fwd_kvcache_noalloc: cannot identify the current device");
    cudaGetLastError();
    return 2;
  }
  if (!ptrs[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fa_host::set_error("fa_fwd_kvcache_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      cudaGetLastError();
      return 2;
    }
    ptrs[dev] = static_cast<unsigned char*>(p);
  }
  *out = ptrs[dev];
  return 0;
}

int decode_run_noalloc(const FaKvcacheArgs& a, int num_splits, cudaStream_t st) {
  const size_t rows = (size_t)a.batch * a.heads * a.seqlen_q;
  const size_t lse_bytes = (rows * num_splits * sizeof(float) + 255) & ~size_t(255);
  const size_t out_bytes = rows * num_splits * (size_t)a.head_dim * sizeof(float);
  FaKvcacheArgs b = a;
  if (num_splits > 1) {
    if (lse_bytes + out_bytes > kNoAllocScratchBytes) {
      fa_host::set_error(
          "fa_fwd_kvcache_noalloc: %d splits of %zu rows need %zu bytes of scratch, the built-in buffer holds %zu; "
          "pass a smaller num_splits or use fa_fwd_kvcache with caller-provided workspaces",
          num_splits, rows, lse_bytes + out_bytes, (size_t)kNoAllocScratchBytes);
      return 1;
    }
    unsigned char* base = nullptr;
    if (noalloc_scratch_ptr(&base)) return 2;
    // Nothing has to be cleared: every (split, row) LSE is written by each launch (-inf for an empty
    // split) and the combine step never reads the partial output of a part whose weight is zero.
    b.lse_accum = reinterpret_cast<float*>(base);
    b.out_accum = reinterpret_cast<float*>(base + lse_bytes);
  }
  return decode_run(b, num_splits, st, /*may_allocate=*/false);
}

}  // namespace fa
