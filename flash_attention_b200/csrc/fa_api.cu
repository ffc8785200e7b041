// C ABI of libfa_b200 (declared in include/fa_b200.h): argument validation, kernel selection,
// launch.  Plays the part of mha_fwd / mha_bwd / mha_fwd_kvcache in
// csrc/flash_attn/flash_api.cpp, minus everything that needs torch (allocation, padding, RNG
// state), which lives in the python shim.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "fa_common.cuh"

namespace fa {
int fwd_generic(const FaFwdArgs& a, cudaStream_t st);
int bwd_pre(const FaBwdArgs& a, int zero_dq, cudaStream_t st);
int bwd_post(const FaBwdArgs& a, cudaStream_t st);
int bwd_generic_main(const FaBwdArgs& a, cudaStream_t st);
int rotary(const FaRotaryArgs& a, cudaStream_t st);
int merge_partial(const FaTensor& acc, float* lse_acc, int64_t lacc_sb, int64_t lacc_sh, const FaTensor& part,
                  const float* lse_part, int64_t lpart_sb, int64_t lpart_sh, int B, int S, int H, int D, int dtype,
                  cudaStream_t st);
int combine(const float* out_parts, const float* lse_parts, const FaTensor& out, float* lse, int lse_pitch, int n_parts,
            int B, int H, int S, int D, int dtype, cudaStream_t st);
int kvcache_prep(const FaKvcacheArgs& a, int q_follows_rows, cudaStream_t st);
// tcgen05 kernels (sm100/)
bool fwd_tc_eligible(const FaFwdArgs& a);
int fwd_tc(const FaFwdArgs& a, cudaStream_t st);
bool bwd_tc_eligible(const FaBwdArgs& a);
int bwd_tc_main(const FaBwdArgs& a, cudaStream_t st);
// fused single-token decode
bool decode_eligible(const FaKvcacheArgs& a);
int decode_plan(const FaKvcacheArgs& a, int num_sms);
int decode_run(const FaKvcacheArgs& a, int num_splits, cudaStream_t st, bool may_allocate = true);
int decode_noalloc_fit(const FaKvcacheArgs& a, int num_splits);
int decode_run_noalloc(const FaKvcacheArgs& a, int num_splits, cudaStream_t st);
size_t decode_noalloc_capacity();
int bwd_dq_tc_main(const FaBwdArgs& a, cudaStream_t st);
int bwd_wide_tc_main(const FaBwdArgs& a, int parts, cudaStream_t st);
// device status word (sm100/status.cu)
int status_peek();
int status_read(bool clear);
int selftest_wait_timeout(long long limit_cycles, int code, cudaStream_t st);
}  // namespace fa

namespace fa_host {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 2;
  }
  return 0;
}
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
int raise_smem_limit(DeviceOnce& once, const void* kernel, int bytes, const char* name) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    dev = -1;
  }
  DeviceOnce probe = once;
  if (!device_once_needed(probe, dev)) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    set_error("%s: cannot reserve %d bytes of shared memory: %s", name, bytes, cudaGetErrorString(cudaGetLastError()));
    return 2;
  }
  device_once_needed(once, dev);
  return 0;
}
static int env_flag(const char* name) {
  const char* v = getenv(name);
  return v && v[0] && v[0] != '0';
}
}  // namespace fa_host

using fa_host::set_error;

// Which kernels the last fa_fwd / fa_bwd / fa_fwd_kvcache call of this process launched (fa_last_path()).
// Process-wide on purpose: a backward pass runs on an autograd worker thread, not on the caller's.
static const char* volatile g_last_path = "";

static int check_tensor(const FaTensor& t, const char* name) {
  FA_REQUIRE(t.ptr != nullptr, "%s: null pointer", name);
  FA_REQUIRE((reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0, "%s: pointer must be 16-byte aligned", name);
  FA_REQUIRE(t.stride_s % 8 == 0 && t.stride_h % 8 == 0 && t.stride_b % 8 == 0,
             "%s: strides must be multiples of 8 elements", name);
  return 0;
}

static int check_common(int batch, int sq, int sk, int heads, int heads_k, int d, int dtype) {
  FA_REQUIRE(batch > 0, "batch size must be positive");
  FA_REQUIRE(d > 0 && d <= 256, "FlashAttention only supports head dimension at most 256");
  FA_REQUIRE(d % 8 == 0, "head dimension must be a multiple of 8 (the caller pads)");
  FA_REQUIRE(heads > 0 && heads_k > 0 && heads % heads_k == 0,
             "Number of heads in key/value must divide number of heads in query");
  FA_REQUIRE(dtype == FA_DTYPE_FP16 || dtype == FA_DTYPE_BF16, "FlashAttention only support fp16 and bf16 data type");
  FA_REQUIRE(sq >= 0 && sk >= 0, "negative sequence length");
  return 0;
}

// A kernel of an earlier call gave up on a bounded wait: refuse to launch until the caller has read
// (and thereby cleared) the status, instead of returning tensors that no kernel wrote.
static int refuse_if_device_failed() {
  const int code = fa::status_peek();
  if (code) {
    set_error("an earlier kernel on this device gave up on a bounded wait (code %d) and its outputs are incomplete; "
              "call fa_device_status() to read and clear the status before launching again", code);
    return 3;
  }
  return 0;
}

extern "C" {

const char* fa_last_error(void) { return fa_host::g_err; }

const char* fa_last_path(void) { return g_last_path; }

const char* fa_build_info(void) {
  return "libfa_b200 arch=sm_100a kernels=fwd_tc(tcgen05+TMA),bwd_dkdv_tc(tcgen05+TMA),bwd_dq_tc(tcgen05+TMA),bwd_wide_tc(tcgen05+TMA),decode_splitkv(TMA),"
         "fwd_generic(mma.sync),bwd_generic(mma.sync),combine,merge_partial,rotary,bwd_dot_do_o,bwd_convert_dq,kvcache_prep";
}

int fa_device_status(void) { return fa::status_read(true); }

int fa_selftest_wait_timeout(int64_t limit_cycles, fa_stream_t stream) {
  FA_REQUIRE(limit_cycles > 0 && limit_cycles <= 100000000ll, "limit_cycles must be in (0, 1e8]");
  return fa::selftest_wait_timeout(limit_cycles, /*code=*/99, reinterpret_cast<cudaStream_t>(stream));
}

int fa_selftest_device_once(const int32_t* devices, int32_t n, int32_t* needed) {
  FA_REQUIRE(devices && needed && n >= 0, "null pointer");
  fa_host::DeviceOnce once = {};
  for (int i = 0; i < n; ++i) needed[i] = fa_host::device_once_needed(once, devices[i]) ? 1 : 0;
  return 0;
}

int fa_abi_struct_size(int32_t which) {
  switch (which) {
    case 0: return (int)sizeof(FaTensor);
    case 1: return (int)sizeof(FaFwdArgs);
    case 2: return (int)sizeof(FaBwdArgs);
    case 3: return (int)sizeof(FaKvcacheArgs);
    case 4: return (int)sizeof(FaRotaryArgs);
    default: return -1;
  }
}

int fa_fwd_num_splits(int32_t batch, int32_t heads, int32_t seqlen_q, int32_t seqlen_k, int32_t head_dim,
                      int32_t num_sms) {
  // Same search as num_splits_heuristic (flash_api.cpp:206-246) on this library's tile sizes (a work
  // item of the tensor-core kernel is 256 query rows, 128 above head dim 128, and walks 128-key
  // blocks): with enough items to fill 80 % of the SMs do not split; otherwise take the smallest
  // split count within 85 % of the best wave efficiency.
  if (num_sms <= 0) num_sms = fa_host::sm_count();
  const int rows = head_dim > 128 ? 128 : 256;
  const int m_blocks = (seqlen_q + rows - 1) / rows, n_blocks = (seqlen_k + 127) / 128;
  const int ctas = batch * heads * m_blocks;
  if (ctas >= 0.8f * num_sms) return 1;
  int max_splits = 128;
  if (num_sms < max_splits) max_splits = num_sms;
  if (n_blocks < max_splits) max_splits = n_blocks;
  if (max_splits < 1) max_splits = 1;
  auto blocks_per = [&](int s) { return (n_blocks + s - 1) / s; };
  float best = 0.f;
  float eff[129];
  for (int s = 1; s <= max_splits; ++s) {
    bool eligible = s == 1 || blocks_per(s) != blocks_per(s - 1);
    if (!eligible) {
      eff[s] = 0.f;
      continue;
    }
    float waves = float(ctas) * s / num_sms;
    float e = waves / ceilf(waves);
    eff[s] = e;
    if (e > best) best = e;
  }
  for (int s = 1; s <= max_splits; ++s)
    if (eff[s] >= 0.85f * best && eff[s] > 0.f) return s;
  return 1;
}

int64_t fa_bwd_workspace_bytes(int32_t batch, int32_t seqlen_q, int32_t heads, int32_t head_dim, int32_t total_q,
                               int32_t is_varlen) {
  // fp32 rows in the layout of dq, used by the any-shape kernel only (the tensor-core kernels
  // write dq directly and leave the workspace untouched)
  int64_t rows = is_varlen ? (int64_t)total_q : (int64_t)batch * seqlen_q;
  return rows * heads * head_dim * (int64_t)sizeof(float);
}

int fa_fwd(const FaFwdArgs* a, fa_stream_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  FA_REQUIRE(a != nullptr, "null arguments");
  if (check_common(a->batch, a->seqlen_q, a->seqlen_k, a->heads, a->heads_k, a->head_dim, a->dtype)) return 1;
  if (check_tensor(a->q, "q") || check_tensor(a->k, "k") || check_tensor(a->v, "v") || check_tensor(a->out, "out"))
    return 1;
  FA_REQUIRE(a->softmax_lse != nullptr, "softmax_lse: null pointer");
  FA_REQUIRE((a->cu_seqlens_q == nullptr) == (a->cu_seqlens_k == nullptr),
             "cu_seqlens_q and cu_seqlens_k must be given together");
  FA_REQUIRE(a->p_dropout >= 0.f && a->p_dropout < 1.f, "p_dropout must be in [0, 1)");
  FA_REQUIRE(a->num_splits <= 128, "num_splits > 128 not supported");
  if (a->num_splits > 1) {
    FA_REQUIRE(a->lse_accum && a->out_accum, "split-KV needs lse_accum and out_accum");
    FA_REQUIRE(!a->cu_seqlens_q, "split-KV is not available for packed variable-length input");
    FA_REQUIRE(a->p_dropout == 0.f, "split-KV does not support dropout");
  }
  if (a->block_table) {
    FA_REQUIRE(a->page_block_size > 0 && a->page_block_size % 64 == 0, "Paged KV cache block size must be divisible by 64");
    FA_REQUIRE(a->block_table_stride > 0 &&
                   (int64_t)a->block_table_stride * a->page_block_size >= a->seqlen_k,
               "a row of block_table must cover seqlen_k keys");
    FA_REQUIRE(!a->cu_seqlens_k && !a->kv_batch_idx && !a->s_dmask,
               "paged K/V is not combined with cu_seqlens_k, kv_batch_idx or a returned probability matrix");
  }
  if (a->seqlen_q == 0 || a->batch == 0) return 0;
  if (refuse_if_device_failed()) return 3;
  int rc;
  if (!fa_host::env_flag("FA_B200_FORCE_GENERIC") && fa::fwd_tc_eligible(*a)) {
    g_last_path = a->num_splits > 1 ? "fwd_tc+combine" : "fwd_tc";
    rc = fa::fwd_tc(*a, st);
  } else {
    g_last_path = a->num_splits > 1 ? "fwd_generic+combine" : "fwd_generic";
    rc = fa::fwd_generic(*a, st);
  }
  if (rc) return rc;
  if (a->num_splits > 1)
    return fa::combine(a->out_accum, a->lse_accum, a->out, a->softmax_lse, a->lse_seqlen, a->num_splits, a->batch,
                       a->heads, a->seqlen_q, a->head_dim, a->dtype, st);
  return 0;
}

int fa_bwd(const FaBwdArgs* a, fa_stream_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  FA_REQUIRE(a != nullptr, "null arguments");
  if (check_common(a->batch, a->seqlen_q, a->seqlen_k, a->heads, a->heads_k, a->head_dim, a->dtype)) return 1;
  if (check_tensor(a->q, "q") || check_tensor(a->k, "k") || check_tensor(a->v, "v") || check_tensor(a->out, "out") ||
      check_tensor(a->dout, "dout") || check_tensor(a->dq, "dq"))
    return 1;
  if (!a->accumulate_dkv) {
    if (check_tensor(a->dk, "dk") || check_tensor(a->dv, "dv")) return 1;
  } else {
    FA_REQUIRE(a->dk_accum && a->dv_accum, "accumulate_dkv needs dk_accum and dv_accum");
  }
  FA_REQUIRE(a->softmax_lse && a->softmax_d && a->dq_accum, "softmax_lse, softmax_d and dq_accum are required");
  FA_REQUIRE((a->cu_seqlens_q == nullptr) == (a->cu_seqlens_k == nullptr),
             "cu_seqlens_q and cu_seqlens_k must be given together");
  FA_REQUIRE(a->p_dropout >= 0.f && a->p_dropout < 1.f, "p_dropout must be in [0, 1)");
  FA_REQUIRE(a->d_seqlen >= a->seqlen_q, "softmax_d row pitch is smaller than seqlen_q");
  if (a->seqlen_q == 0 || a->batch == 0) return 0;
  if (refuse_if_device_failed()) return 3;
  const bool tc = a->seqlen_k > 0 && !fa_host::env_flag("FA_B200_FORCE_GENERIC") && fa::bwd_tc_eligible(*a);
  const int parts = a->parts == 0 ? 3 : a->parts;  // bit 0: dot(dO, O) and dQ, bit 1: dK and dV
  FA_REQUIRE(parts >= 1 && parts <= 3, "parts must be 0 (everything), 1 (preprocess and dQ) or 2 (dK and dV)");
  FA_REQUIRE(parts == 3 || tc, "a backward pass can only be split in parts on the tensor-core path");
  // the tensor-core path writes dq directly (two kernels: dK / dV per key block, dQ per query block)
  int rc = (parts & 1) ? fa::bwd_pre(*a, tc ? 0 : 1, st) : 0;
  if (rc) return rc;
  g_last_path = !tc ? "bwd_generic" : (a->head_dim > 128 ? "bwd_wide_tc" : "bwd_tc+bwd_dq_tc");
  if (tc) {
    if (a->head_dim > 128) return fa::bwd_wide_tc_main(*a, parts, st);  // one pass per output
    if (parts & 2) rc = fa::bwd_tc_main(*a, st);
    if (!rc && (parts & 1)) rc = fa::bwd_dq_tc_main(*a, st);
    return rc;
  }
  if (a->seqlen_k > 0) {
    rc = fa::bwd_generic_main(*a, st);
    if (rc) return rc;
  }
  return fa::bwd_post(*a, st);
}

static int kvcache_checks(const FaKvcacheArgs* a) {
  FA_REQUIRE(a != nullptr, "null arguments");
  if (check_common(a->batch, a->seqlen_q, a->seqlen_cache, a->heads, a->heads_k, a->head_dim, a->dtype)) return 1;
  FA_REQUIRE(a->batch_cache > 0, "batch size must be postive");
  FA_REQUIRE(a->num_splits >= 0 && a->num_splits <= 128, "num_splits > 128 not supported");
  if (a->knew.ptr) {
    FA_REQUIRE(a->vnew.ptr != nullptr, "If key is supplied, value must also be passed in");
    FA_REQUIRE(a->cache_seqlens != nullptr, "If key is supplied, seqlens_k must also be passed in");
    FA_REQUIRE(a->seqlen_q <= a->seqlen_cache, "If key is supplied, it must have seqlen <= the seqlen of the KV cache");
  }
  if (a->rotary_cos) {
    FA_REQUIRE(a->knew.ptr != nullptr, "If rotary cos/sin are provided, new key / value to be appended to KV cache must also be provided");
    FA_REQUIRE(a->rotary_sin != nullptr, "rotary_sin is required with rotary_cos");
    FA_REQUIRE(a->rotary_dim > 0 && a->rotary_dim <= a->head_dim, "rotary_dim must be <= headdim");
    FA_REQUIRE(a->rotary_dim % 16 == 0, "Only rotary dimensions divisible by 16 are currently supported");
    FA_REQUIRE(a->seqlen_ro >= a->seqlen_cache, "cos/sin seqlen must be at least the seqlen of KV cache");
  }
  if (a->block_table) {
    FA_REQUIRE(a->cache_batch_idx == nullptr, "Paged KVcache does not support cache_batch_idx");
    FA_REQUIRE(a->page_block_size > 0 && a->page_block_size % 64 == 0, "Paged KV cache block size must be divisible by 64");
    FA_REQUIRE(a->block_table_stride > 0 && a->seqlen_cache % a->page_block_size == 0 &&
                   a->seqlen_cache / a->page_block_size <= a->block_table_stride,
               "seqlen_cache must be (pages per sequence) * page_block_size, within one row of block_table");
  } else if (!a->cache_batch_idx) {
    FA_REQUIRE(a->batch_cache >= a->batch, "the KV cache holds fewer sequences than q");
  }
  return 0;
}

int fa_kvcache_plan(const FaKvcacheArgs* a, int32_t num_sms, int64_t* lse_accum_bytes, int64_t* out_accum_bytes) {
  if (kvcache_checks(a)) return -1;
  if (num_sms <= 0) num_sms = fa_host::sm_count();
  int splits;
  if (!fa_host::env_flag("FA_B200_FORCE_GENERIC") && fa::decode_eligible(*a)) {
    splits = fa::decode_plan(*a, num_sms);
  } else {
    splits = a->num_splits;
    if (splits == 0) splits = fa_fwd_num_splits(a->batch, a->heads, a->seqlen_q, a->seqlen_cache, a->head_dim, num_sms);
  }
  if (splits < 1) splits = 1;
  int64_t rows = (int64_t)a->batch * a->heads * a->seqlen_q;
  if (lse_accum_bytes) *lse_accum_bytes = splits > 1 ? rows * splits * (int64_t)sizeof(float) : 0;
  if (out_accum_bytes) *out_accum_bytes = splits > 1 ? rows * splits * a->head_dim * (int64_t)sizeof(float) : 0;
  return splits;
}

int fa_fwd_kvcache(const FaKvcacheArgs* a, fa_stream_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kvcache_checks(a)) return 1;
  if (check_tensor(a->q, "q") || check_tensor(a->kcache, "kcache") || check_tensor(a->vcache, "vcache") ||
      check_tensor(a->out, "out"))
    return 1;
  int splits = fa_kvcache_plan(a, 0, nullptr, nullptr);
  if (splits < 0) return 1;
  if (splits > 1) FA_REQUIRE(a->lse_accum && a->out_accum, "split-KV needs lse_accum and out_accum");
  if (a->seqlen_q == 0) return 0;
  if (refuse_if_device_failed()) return 3;
  if (!fa_host::env_flag("FA_B200_FORCE_GENERIC") && fa::decode_eligible(*a)) {
    g_last_path = splits > 1 ? "decode+combine" : "decode";
    return fa::decode_run(*a, splits, st);
  }
  g_last_path = splits > 1 ? "kvcache_prep+fwd_generic+combine" : "kvcache_prep+fwd_generic";

  // General path: append/rotate in a first launch, then the any-shape forward on the cache.
  const bool causal_or_local = a->window_left >= 0 || a->window_right >= 0;
  FA_REQUIRE(!a->rotary_cos || a->q_rotated, "rotary needs the q_rotated scratch buffer");
  int rc = fa::kvcache_prep(*a, (causal_or_local && !a->q_rows_share_position) ? 1 : 0, st);
  if (rc) return rc;
  FaFwdArgs f;
  memset(&f, 0, sizeof(f));
  if (a->rotary_cos) {
    f.q.ptr = a->q_rotated;
    f.q.stride_h = a->head_dim;
    f.q.stride_s = (int64_t)a->heads * a->head_dim;
    f.q.stride_b = (int64_t)a->seqlen_q * a->heads * a->head_dim;
  } else {
    f.q = a->q;
  }
  f.k = a->kcache;
  f.v = a->vcache;
  f.out = a->out;
  f.softmax_lse = a->softmax_lse;
  f.lse_seqlen = a->seqlen_q;
  f.batch = a->batch;
  f.seqlen_q = a->seqlen_q;
  f.seqlen_k = a->seqlen_cache;
  f.heads = a->heads;
  f.heads_k = a->heads_k;
  f.head_dim = a->head_dim;
  f.dtype = a->dtype;
  f.softmax_scale = a->softmax_scale;
  f.window_left = a->window_left;
  f.window_right = a->window_right;
  f.seqused_k = a->cache_seqlens;
  f.seqused_k_extra = a->knew.ptr ? a->seqlen_new : 0;
  f.kv_batch_idx = a->cache_batch_idx;
  f.block_table = a->block_table;
  f.block_table_stride = a->block_table_stride;
  f.page_block_size = a->page_block_size;
  f.num_splits = splits;
  f.lse_accum = a->lse_accum;
  f.out_accum = a->out_accum;
  rc = fa::fwd_generic(f, st);
  if (rc) return rc;
  if (splits > 1)
    return fa::combine(a->out_accum, a->lse_accum, a->out, a->softmax_lse, a->seqlen_q, splits, a->batch, a->heads,
                       a->seqlen_q, a->head_dim, a->dtype, st);
  return 0;
}

int fa_fwd_kvcache_noalloc(const FaKvcacheArgs* a, fa_stream_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kvcache_checks(a)) return 1;
  if (check_tensor(a->q, "q") || check_tensor(a->kcache, "kcache") || check_tensor(a->vcache, "vcache") ||
      check_tensor(a->out, "out"))
    return 1;
  FA_REQUIRE(fa::decode_eligible(*a),
             "fa_fwd_kvcache_noalloc only covers the single-token decode shape: seqlen_q * heads / heads_k <= 16, head_dim 64 "
             "or 128, no window, at most one new token");
  FA_REQUIRE(a->softmax_lse != nullptr, "softmax_lse: null pointer");
  int splits = fa::decode_plan(*a, fa_host::sm_count());
  if (splits < 1) splits = 1;
  // asked to choose: choose among the split counts whose partials fit the built-in buffer
  if (a->num_splits == 0) splits = fa::decode_noalloc_fit(*a, splits);
  if (a->seqlen_q == 0) return 0;
  if (refuse_if_device_failed()) return 3;
  g_last_path = splits > 1 ? "decode+combine" : "decode";
  return fa::decode_run_noalloc(*a, splits, st);
}

int64_t fa_noalloc_scratch_bytes(void) { return (int64_t)fa::decode_noalloc_capacity(); }

int fa_combine(const float* out_parts, const float* lse_parts, void* out, float* lse, int32_t n_parts, int64_t rows,
               int32_t head_dim, int64_t out_row_stride, int32_t dtype, fa_stream_t stream) {
  FA_REQUIRE(out_parts && lse_parts && out, "null pointer");
  FA_REQUIRE(n_parts >= 1 && n_parts <= 128, "n_parts must be in [1, 128]");
  FA_REQUIRE(head_dim % 8 == 0 && head_dim <= 256, "head_dim must be a multiple of 8, at most 256");
  FA_REQUIRE(rows < (1ll << 31), "too many rows");
  FaTensor o{out, 0, out_row_stride, 0};
  return fa::combine(out_parts, lse_parts, o, lse, (int)rows, n_parts, 1, 1, (int)rows, head_dim, dtype,
                     reinterpret_cast<cudaStream_t>(stream));
}

int fa_merge_partial(const FaTensor* acc, float* lse_acc, int64_t lse_acc_stride_b, int64_t lse_acc_stride_h,
                     const FaTensor* part, const float* lse_part, int64_t lse_part_stride_b, int64_t lse_part_stride_h,
                     int32_t batch, int32_t seqlen, int32_t heads, int32_t head_dim, int32_t dtype, fa_stream_t stream) {
  FA_REQUIRE(acc && part && acc->ptr && part->ptr && lse_acc && lse_part, "null pointer");
  FA_REQUIRE(dtype == FA_DTYPE_FP16 || dtype == FA_DTYPE_BF16, "FlashAttention only support fp16 and bf16 data type");
  FA_REQUIRE(batch >= 0 && seqlen >= 0 && heads > 0, "bad sizes");
  FA_REQUIRE(head_dim % 8 == 0 && head_dim > 0 && head_dim <= 256, "head_dim must be a multiple of 8, at most 256");
  FA_REQUIRE((reinterpret_cast<uintptr_t>(acc->ptr) & 15) == 0 && (reinterpret_cast<uintptr_t>(part->ptr) & 7) == 0 &&
                 acc->stride_s % 4 == 0 && acc->stride_h % 4 == 0 && acc->stride_b % 4 == 0 && part->stride_s % 4 == 0 &&
                 part->stride_h % 4 == 0 && part->stride_b % 4 == 0,
             "accumulator rows must be 16-byte aligned, partial rows 8-byte aligned");
  return fa::merge_partial(*acc, lse_acc, lse_acc_stride_b, lse_acc_stride_h, *part, lse_part, lse_part_stride_b,
                           lse_part_stride_h, batch, seqlen, heads, head_dim, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int fa_rotary(const FaRotaryArgs* a, fa_stream_t stream) {
  FA_REQUIRE(a != nullptr, "null arguments");
  FA_REQUIRE(a->dtype == FA_DTYPE_FP16 || a->dtype == FA_DTYPE_BF16, "rotary only supports fp16 and bf16 data type");
  FA_REQUIRE(a->batch >= 0 && a->seqlen >= 0 && a->heads > 0 && a->head_dim > 0, "bad sizes");
  FA_REQUIRE(a->head_dim <= 256, "Only support headdim <= 256");
  FA_REQUIRE(a->rotary_dim >= 0 && a->rotary_dim % 2 == 0, "rotary_dim must be even");
  FA_REQUIRE(a->rotary_dim <= a->head_dim, "rotary_dim must be <= headdim");
  FA_REQUIRE(a->cu_seqlens != nullptr || a->seqlen_ro >= a->seqlen, "seqlen_ro must be >= seqlen");
  FA_REQUIRE(a->seqlen_offsets != nullptr || a->cu_seqlens != nullptr || a->seqlen_offset + a->seqlen <= a->seqlen_ro,
             "seqlen_offsets + seqlen must be <= seqlen_ro");
  const int64_t rows = a->cu_seqlens ? (int64_t)a->total : (int64_t)a->batch * a->seqlen;
  if (rows == 0) return 0;
  FA_REQUIRE(a->x.ptr && a->out.ptr, "x / out: null pointer");
  FA_REQUIRE(a->rotary_dim == 0 || (a->cos && a->sin), "cos / sin: null pointer");
  return fa::rotary(*a, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
