// Host-side construction of TMA tensor maps for (batch, seq, head, dim) operands with arbitrary
// 16-byte-aligned strides.  The driver entry point is resolved at run time so that the library
// links against the CUDA runtime only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../fa_common.cuh"

namespace fa {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// 4-D map with dims (dim, seq, head, batch), 128-byte swizzle, box = 64 elements x box_rows rows.
// Out-of-range elements read as zero.  `rows`/`batches` describe the extent of the tensor: for
// packed variable-length tensors rows = total tokens and batches = 1.
static inline int make_tmap_4d(CUtensorMap* map, const FaTensor& t, int dtype, int64_t rows, int heads, int64_t batches,
                               int head_dim, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    fa_host::set_error("cuTensorMapEncodeTiled is not available from this driver");
    return 1;
  }
  cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batches};
  // strides of dims 1..3 in bytes; a degenerate dim still needs a legal (non-zero, 16 B multiple) stride
  auto legal = [](int64_t elems) { return (cuuint64_t)(elems > 0 ? elems : 8) * 2; };
  cuuint64_t strides[3] = {legal(t.stride_s), legal(t.stride_h), legal(t.stride_b)};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, dtype == FA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fa_host::set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 1;
  }
  return 0;
}

static inline bool tma_compatible(const FaTensor& t) {
  auto ok = [](int64_t s) { return s >= 0 && s % 8 == 0 && s < (1ll << 38); };
  return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && ok(t.stride_s) && ok(t.stride_h) && ok(t.stride_b);
}

}  // namespace fa
