// Host helper: a TMA tensor map over a row-major [rows, dims] bf16 / fp16 matrix with a box of 64 dims x box_rows rows in the
// 128-byte swizzle (the layout of a K-major UMMA operand chunk).  cuTensorMapEncodeTiled is resolved through the runtime so
// that the library does not link against the driver library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dsa {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// false when the map cannot be made (no driver entry point, base not 16-byte aligned, too many rows): callers then use
// their cp.async loaders.  Rows beyond `rows` read as zeros.
inline bool encode_rows_map(const void* base, long long rows, int dims, bool bf16, int box_rows, CUtensorMap* map) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode || (reinterpret_cast<uintptr_t>(base) & 15u) || rows <= 0 || rows > 0x7fffffffLL || box_rows <= 0 || box_rows > 256) return false;
  const cuuint64_t gdims[2] = {static_cast<cuuint64_t>(dims), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(dims) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)}, estr[2] = {1, 1};
  return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace dsa
