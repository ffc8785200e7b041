/*
 * fa_b200.h — C ABI of libfa_b200.so, a Blackwell (sm_100a) exact-attention library.
 *
 * The library replaces the five entry points of the FlashAttention v2.3.3 extension module
 * `flash_attn_2_cuda` (csrc/flash_attn/flash_api.cpp:1281-1288: fwd, varlen_fwd, bwd, varlen_bwd,
 * fwd_kvcache).  Those entry points take torch tensors; this ABI takes what they boil down to:
 * raw device pointers, element strides, sizes and scalars.  Allocation, shape checks that need
 * tensor metadata, head-dim padding and RNG state stay in the host shim (python module
 * `flash_attn_2_cuda` of this repository).
 *
 * Conventions (same as the reference, csrc/flash_attn/flash_api.cpp:21-119):
 *   - q is (batch, seqlen_q, heads, head_dim), k/v are (batch, seqlen_k, heads_k, head_dim); only
 *     the last dimension must be contiguous.  Strides are in ELEMENTS and 64-bit.
 *   - varlen: tensors are (total_tokens, heads, head_dim) and cu_seqlens_* hold batch+1 int32
 *     prefix sums on the device; batch strides are ignored.
 *   - head_dim must be a multiple of 8 and <= 256 (the shim pads, flash_api.cpp:313-322).
 *   - softmax_lse is fp32 (batch, heads, seqlen_q) [varlen: (batch, heads, max_seqlen_q)], natural
 *     log of the row sum of exp(scale * q.k), +inf for a row with no visible key
 *     (csrc/flash_attn/src/flash_fwd_kernel.h:505-516).
 *   - masks are aligned to the bottom-right corner: key j is visible to query i iff
 *       i + shift - window_left <= j <= i + shift + window_right,  shift = seqlen_k - seqlen_q
 *     with a negative window meaning "unbounded on that side" (csrc/flash_attn/src/softmax.h:142-179).
 *     `causal` is window_right = 0.
 *   - every function enqueues work on `stream` and returns without synchronising; 0 = success,
 *     1 = invalid arguments, 2 = a CUDA call failed, 3 = refused because an earlier kernel gave up on
 *     a bounded wait (see fa_device_status); fa_last_error() describes the failure (the shim raises
 *     RuntimeError, mirroring TORCH_CHECK in the reference).
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* fa_stream_t; /* a cudaStream_t */

enum { FA_DTYPE_FP16 = 0, FA_DTYPE_BF16 = 1 };

/* One strided (batch, seq, head, dim) operand: element strides, dim stride is 1. */
typedef struct FaTensor {
  void* ptr;
  int64_t stride_b; /* batch stride (ignored for varlen) */
  int64_t stride_s; /* row (token) stride */
  int64_t stride_h; /* head stride */
} FaTensor;

/* Forward.  Replaces mha_fwd (flash_api.cpp:248-424) and mha_varlen_fwd (flash_api.cpp:426-585). */
typedef struct FaFwdArgs {
  FaTensor q, k, v, out;
  float* softmax_lse;       /* (batch, heads, lse_seqlen) fp32 */
  int32_t lse_seqlen;       /* row pitch of softmax_lse: seqlen_q, or max_seqlen_q for varlen */
  int32_t batch, seqlen_q, seqlen_k, heads, heads_k, head_dim;
  int32_t dtype;            /* FA_DTYPE_* */
  float softmax_scale;
  int32_t window_left, window_right; /* < 0: unbounded */
  /* varlen (both NULL for fixed-length batches); seqlen_q/seqlen_k are then the maxima */
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  int32_t total_q, total_k; /* rows of the packed tensors (varlen only) */
  /* per-batch key lengths that are NOT cumulative (KV cache, flash_api.cpp:1198-1206); may be NULL */
  const int32_t* seqused_k;
  int32_t seqused_k_extra;  /* added to every seqused_k entry (rows appended to the cache by this call) */
  /* optional gather of the k/v batch index (cache_batch_idx, flash_api.cpp:1234-1240) */
  const int32_t* kv_batch_idx;
  /* dropout (flash_api.cpp:391-406).  p_dropout = probability of dropping. */
  float p_dropout;
  uint64_t rng_seed, rng_offset;
  /* optional (batch, heads, sdmask_rows, sdmask_cols) tensor of q's dtype receiving the softmax
     probabilities with the sign bit set where the entry was dropped (flash_api.cpp:351-354). */
  void* s_dmask;
  int32_t sdmask_rows, sdmask_cols;
  /* split-KV (flash_api.cpp:373-389): num_splits <= 1 means one pass.  Workspaces are fp32:
     lse_accum (num_splits, batch, heads, seqlen_q), out_accum (num_splits, batch, heads, seqlen_q, head_dim). */
  int32_t num_splits;
  float* lse_accum;
  float* out_accum;
  /* Mask shift override used by the context-parallel ring: when use_mask_shift != 0 the `shift`
     of the mask rule above is mask_shift instead of seqlen_k - seqlen_q (no reference counterpart;
     the reference has no ring attention). */
  int32_t use_mask_shift;
  int32_t mask_shift;
  /* Paged K/V (no counterpart in this version of the reference; the nearest thing is the kv_batch_idx
     gather of flash_api.cpp:1234-1240).  When block_table != NULL, k / v are pools of pages
     (num_pages, page_block_size, heads_k, head_dim) addressed with stride_b = page pitch, and key j of
     sequence b lives in row j % page_block_size of page block_table[b * block_table_stride +
     j / page_block_size].  page_block_size must be a multiple of 64; not combined with cu_seqlens_k,
     kv_batch_idx or s_dmask.  Such a call runs on the any-shape kernel. */
  const int32_t* block_table;
  int32_t block_table_stride;
  int32_t page_block_size;
} FaFwdArgs;

/* Backward.  Replaces mha_bwd (flash_api.cpp:609-811) and mha_varlen_bwd (flash_api.cpp:813-1036),
   i.e. the three launches dot_do_o -> dq_dk_dv -> convert_dq of
   csrc/flash_attn/src/flash_bwd_launch_template.h:47-90.  Without dropout the launches are
   dot_do_o -> dK/dV kernel -> dQ kernel (head dims up to 128) or dot_do_o -> dV pass -> dK pass ->
   dQ pass (129..256) instead: dq is written directly, without atomics, and dq_accum is not touched. */
typedef struct FaBwdArgs {
  FaTensor q, k, v, out, dout, dq, dk, dv;
  const float* softmax_lse; /* from the forward, same layout */
  int32_t lse_seqlen;
  float* softmax_d;         /* (batch, heads, d_seqlen) fp32 out: rowsum(dO * O) */
  int32_t d_seqlen;         /* row pitch of softmax_d (seqlen_q rounded up to 128) */
  float* dq_accum;          /* fp32 workspace, fa_bwd_workspace_bytes() bytes, need not be zeroed (used by the any-shape kernel) */
  int32_t batch, seqlen_q, seqlen_k, heads, heads_k, head_dim;
  int32_t dtype;
  float softmax_scale;
  int32_t window_left, window_right;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  int32_t total_q, total_k;
  float p_dropout;
  uint64_t rng_seed, rng_offset;
  int32_t use_mask_shift;
  int32_t mask_shift;
  /* when non-zero dk/dv are ACCUMULATED into fp32 tensors dk_accum/dv_accum of shape
     (batch|total_k, seqlen_k, heads_k, head_dim) instead of being stored (ring backward). */
  int32_t accumulate_dkv;
  float* dk_accum;
  float* dv_accum;
  /* Run only part of the pass (tensor-core path only; no counterpart in the reference): 0 = everything,
     1 = dot(dO, O) into softmax_d and dQ, 2 = dK and dV (softmax_d must hold the result of an earlier
     call with 1).  The ring backward uses it to receive the travelling dK / dV accumulators while dQ of
     the same step is being computed. */
  int32_t parts;
  /* != 0: dq must be bit-reproducible from run to run.  The tensor-core kernels always are (nothing is
     accumulated atomically).  The any-shape kernel adds its dq tiles into dq_accum with fp32 atomics,
     one key block per CTA; with this flag it is launched once per key block, so that every dq value
     receives its terms in key order (slower: seqlen_k / 64 launches). */
  int32_t deterministic;
} FaBwdArgs;

/* KV-cache decode.  Replaces mha_fwd_kvcache (flash_api.cpp:1038-1279). */
typedef struct FaKvcacheArgs {
  FaTensor q, kcache, vcache, out;
  FaTensor knew, vnew;      /* ptr NULL when there is nothing to append */
  float* softmax_lse;       /* (batch, heads, seqlen_q) */
  int32_t batch, batch_cache, seqlen_q, seqlen_cache, seqlen_new, heads, heads_k, head_dim;
  int32_t dtype;
  float softmax_scale;
  int32_t window_left, window_right;
  const int32_t* cache_seqlens;   /* (batch) int32 or NULL (= seqlen_cache) */
  const int32_t* cache_batch_idx; /* (batch) int32 or NULL */
  const void* rotary_cos;         /* (seqlen_ro, rotary_dim/2) of q's dtype or NULL */
  const void* rotary_sin;
  int32_t rotary_dim, seqlen_ro, rotary_interleaved;
  /* q rows of one KV head that were folded into the row dimension by the caller
     (flash_api.cpp:1096-1104); rotary then uses one position for all rows. */
  int32_t q_rows_share_position;
  int32_t num_splits;             /* 0 = choose, 1 = none, <= 128 */
  /* workspaces, fa_kvcache_workspace_bytes() */
  float* lse_accum;
  float* out_accum;
  void* q_rotated;                /* scratch for rotated q when the generic path is taken, or NULL */
  /* Paged cache: block_table != NULL makes kcache / vcache pools of pages (batch_cache = number of pages,
     page_block_size rows each, stride_b = page pitch); key j of sequence b is row j % page_block_size of
     page block_table[b * block_table_stride + j / page_block_size]; seqlen_cache is then the capacity
     per sequence, (entries per row of the table) * page_block_size.  page_block_size % 64 == 0;
     cache_batch_idx must be NULL.  The fused decode kernel fetches one TMA box per 64 keys from the
     page the table names; new tokens are appended through the table as well. */
  const int32_t* block_table;
  int32_t block_table_stride;
  int32_t page_block_size;
} FaKvcacheArgs;

/* flash_attn_2_cuda.fwd / varlen_fwd */
int fa_fwd(const FaFwdArgs* args, fa_stream_t stream);
/* flash_attn_2_cuda.bwd / varlen_bwd */
int fa_bwd(const FaBwdArgs* args, fa_stream_t stream);
/* flash_attn_2_cuda.fwd_kvcache */
int fa_fwd_kvcache(const FaKvcacheArgs* args, fa_stream_t stream);

/* Split-KV decode for callers that cannot allocate device memory.  (No counterpart in the
   reference, whose mha_fwd_kvcache always allocates its split workspaces through torch.)
   Some hosts of this library must not call cudaMalloc at all at decode time: an inference server
   whose memory pool owns the whole device, a real-time loop that may not block on the allocator, a
   plugin running inside someone else's pre-sized arena.  fa_fwd_kvcache needs lse_accum / out_accum
   workspaces from such a caller; this variant does not.  The per-split partial results go to a
   fixed buffer that is part of the library's device image (fa_noalloc_scratch_bytes() bytes, 24 MiB,
   reserved on every GPU that loads the library until the process exits).  The caller still passes
   q, the caches, the optional new token / rotary tables and out / softmax_lse; lse_accum, out_accum
   and q_rotated in the argument struct are ignored.
   Limits and rules:
     - only the single-token decode shape (seqlen_q * heads / heads_k <= 16, head_dim 64 or 128, no
       window, at most one new token); anything else is refused with status 1;
     - with rows = batch * heads * seqlen_q, the partials of a call with S > 1 splits take
       round_up(S * rows * 4, 256) + S * rows * head_dim * 4 bytes.  With num_splits = 0 (choose) the
       library picks the largest split count of its plan that fits the buffer (one split always fits:
       it writes no partials); an explicit num_splits that does not fit is refused with a message
       saying so;
     - the first call on each device looks up the buffer's address (with that device current); make
       that first call outside any stream capture;
     - all calls share the one buffer, which keeps whatever the previous call left in it.  Nothing in
       it needs clearing between calls (every launch rewrites every value it later reads), but two
       calls whose kernels overlap on the GPU (different streams) race on it: serialise them;
     - the call itself performs no cudaMalloc / cudaFree or other allocating call. */
int fa_fwd_kvcache_noalloc(const FaKvcacheArgs* args, fa_stream_t stream);
int64_t fa_noalloc_scratch_bytes(void);

/* Number of KV splits fa_fwd would like for these sizes (num_splits_heuristic, flash_api.cpp:206-246).
   The caller sizes lse_accum/out_accum from it and passes it back in FaFwdArgs.num_splits. */
int fa_fwd_num_splits(int32_t batch, int32_t heads, int32_t seqlen_q, int32_t seqlen_k, int32_t head_dim,
                      int32_t num_sms);
/* Splits and workspace sizes of fa_fwd_kvcache for these arguments (pointers may be NULL);
   returns the number of splits that the call will use and stores the byte sizes. */
int fa_kvcache_plan(const FaKvcacheArgs* args, int32_t num_sms, int64_t* lse_accum_bytes, int64_t* out_accum_bytes);
/* Bytes of FaBwdArgs.dq_accum (dq_accum of flash_api.cpp:735-739, 950-961). */
int64_t fa_bwd_workspace_bytes(int32_t batch, int32_t seqlen_q, int32_t heads, int32_t head_dim, int32_t total_q,
                               int32_t is_varlen);

/* Merge partial attention results by their log-sum-exp (combine_attn_seqk_parallel,
   csrc/flash_attn/src/flash_fwd_kernel.h:1169-1327).  out_parts (n_parts, rows, head_dim) fp32 and
   lse_parts (n_parts, rows) fp32 -> out (rows, head_dim) of `dtype` with row stride out_row_stride,
   lse (rows) fp32. */
int fa_combine(const float* out_parts, const float* lse_parts, void* out, float* lse, int32_t n_parts, int64_t rows,
               int32_t head_dim, int64_t out_row_stride, int32_t dtype, fa_stream_t stream);

/* In-place merge of one more partial result into a running accumulator, the per-step update of
   context-parallel ring attention (same math as the split combine above, one part at a time; the
   reference has no multi-GPU attention and therefore no counterpart):
     acc (batch, seqlen, heads, head_dim) fp32 and lse_acc (batch, heads, seqlen) fp32 are updated with
     part (same shape, `dtype`) and lse_part; strides in elements, head_dim / seqlen contiguous.
   An LSE of +inf or -inf marks a row without keys; lse_acc uses -inf for "still empty". */
int fa_merge_partial(const FaTensor* acc, float* lse_acc, int64_t lse_acc_stride_b, int64_t lse_acc_stride_h,
                     const FaTensor* part, const float* lse_part, int64_t lse_part_stride_b, int64_t lse_part_stride_h,
                     int32_t batch, int32_t seqlen, int32_t heads, int32_t head_dim, int32_t dtype, fa_stream_t stream);

/* Rotary position embedding, the step before attention.  Replaces apply_rotary
   (flash_attn/ops/triton/rotary.py:143-240, kernel :17-140) behind apply_rotary_emb,
   apply_rotary_emb_qkv_ and apply_rotary_emb_kv_ (flash_attn/layers/rotary.py:35-330).
   x and out are (batch, seqlen, heads, head_dim), or packed (total, heads, head_dim) with
   cu_seqlens (stride_b unused); out may be x.  cos / sin are (seqlen_ro, rotary_dim / 2) tables of
   the same 16-bit type as x, contiguous.  Row s of sequence b uses table row
   s + seqlen_offsets[b] (or + seqlen_offset); rows past the tables are left unrotated. */
typedef struct FaRotaryArgs {
  FaTensor x, out;
  const void* cos;
  const void* sin;
  const int32_t* seqlen_offsets; /* (batch) or NULL */
  const int32_t* cu_seqlens;     /* (batch + 1) or NULL */
  int32_t batch, seqlen, heads, head_dim; /* seqlen: max_seqlen for packed input */
  int32_t total;                 /* rows of a packed input */
  int32_t rotary_dim, seqlen_ro;
  int32_t seqlen_offset;
  int32_t dtype;
  int32_t interleaved;           /* pairs (2i, 2i+1) instead of (i, i + rotary_dim/2) */
  int32_t conjugate;             /* rotate by the negative angle: the backward */
} FaRotaryArgs;
int fa_rotary(const FaRotaryArgs* args, fa_stream_t stream);

/* sizeof() of the argument structs as compiled (0: FaTensor, 1: FaFwdArgs, 2: FaBwdArgs,
   3: FaKvcacheArgs, 4: FaRotaryArgs), so that a foreign-function binding can verify its own layout. */
int fa_abi_struct_size(int32_t which);

/* Message for the last non-zero status returned on this thread. */
const char* fa_last_error(void);
/* Names of the kernels that the last fa_fwd / fa_bwd / fa_fwd_kvcache[_noalloc] call of this process
   (whichever thread made it) launched, e.g. "fwd_tc", "fwd_generic+combine", "bwd_tc+bwd_dq_tc", "bwd_wide_tc", "decode+combine"
   (no counterpart in the reference; tests use it to pin a case to the kernel it is meant to cover). */
const char* fa_last_path(void);
/* Compile-time facts: "sm_100a", kernel list, build flags. */
const char* fa_build_info(void);
/* Device-side status word of the tensor-core and decode kernels: 0 = ok, otherwise the code of the
   first bounded wait that gave up (the kernels never spin forever; the reference has no such word,
   its kernels use unbounded __syncthreads / cp.async waits).  The word is sticky: once set, kernels
   of later calls wind down without writing their outputs, and fa_fwd / fa_bwd / fa_fwd_kvcache /
   fa_fwd_kvcache_noalloc return status 3 without launching (they see the word through a mirror in
   mapped host memory, without synchronising).  fa_device_status() synchronises the current device,
   returns the word and clears it, after which calls are accepted again. */
int fa_device_status(void);
/* Self-tests of the failure path (no counterpart in the reference).  fa_selftest_wait_timeout
   launches one warp that waits, for at most limit_cycles SM cycles, on a barrier nobody arrives at,
   and so sets the status word to 99 exactly as a stuck pipeline would; nothing faults or hangs.
   fa_selftest_device_once replays the per-device "raise the shared-memory limit once" bookkeeping of
   the kernel launchers on a list of device ordinals (host only): needed[i] = 1 where call i would
   have configured its device. */
int fa_selftest_wait_timeout(int64_t limit_cycles, fa_stream_t stream);
int fa_selftest_device_once(const int32_t* devices, int32_t n, int32_t* needed);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
