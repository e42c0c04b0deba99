// Host helper: encode 2-D tiled TMA descriptors through the driver entry point
// fetched at run time (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace orinfer {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_encodeTiled runtime_tma_encoder();

// Row-major [rows, cols] matrix of `elem_bytes`-wide elements; box = [box_rows, box_cols];
// 128-byte swizzle (box_cols * elem_bytes must be 128); out-of-range reads give zeros.
inline bool make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType type,
                         uint32_t elem_bytes, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                         uint32_t box_rows, uint32_t box_cols) {
  PFN_encodeTiled enc = runtime_tma_encoder();
  if (!enc) return false;
  if (reinterpret_cast<uintptr_t>(base) % 16 || row_stride_bytes % 16) return false;
  if (box_cols * elem_bytes != 128 || box_rows > 256) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, type, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace orinfer
