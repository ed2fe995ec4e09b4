// Host helpers that encode the TMA tensor maps of the fused kernels (cuTensorMapEncodeTiled, fetched from the driver
// through the runtime so the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "internal.h"

namespace fdb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// (rows, heads, 64) tensor with element strides -> 3-D map (d, head, row), box 64 x 1 x box_rows.
// bf16: 128-byte rows, 128-byte swizzle.  e4m3 (`f8`): 64-byte rows, 64-byte swizzle.
inline int make_map_rows(CUtensorMap* m, const void* base, int64_t rows, int heads, int64_t row_stride,
                         int64_t head_stride, int box_rows, bool f8, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(FDB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t esz = f8 ? 1 : 2;
  const cuuint64_t dims[3] = {64, (cuuint64_t)heads, (cuuint64_t)rows};
  const cuuint64_t strides[2] = {(cuuint64_t)head_stride * esz, (cuuint64_t)row_stride * esz};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(m, f8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        f8 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FDB_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  return FDB_OK;
}

// expanded table (heads, xrows, 64) contiguous -> 3-D map (d, row, head), box 64 x 256 x 1
inline int make_map_table(CUtensorMap* m, const void* base, int xrows, int heads, bool f8, const char* what,
                          int box_rows = kWindow) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(FDB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t row = f8 ? 64 : 128;
  const cuuint64_t dims[3] = {64, (cuuint64_t)xrows, (cuuint64_t)heads};
  const cuuint64_t strides[2] = {row, (cuuint64_t)xrows * row};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(m, f8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        f8 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FDB_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  return FDB_OK;
}

}  // namespace fdb
