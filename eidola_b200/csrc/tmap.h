// Tiled TMA tensor-map creation through the driver entry point (no link-time dependency on libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "common.h"

namespace eb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor of `rows` x `row_bytes` (row pitch `pitch_bytes`), copied in boxes of `box_rows` rows by
// 128 bytes with the 128-byte swizzle.  elem: CU_TENSOR_MAP_DATA_TYPE_UINT8 (row_bytes elements per row) or
// CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 (row_bytes/2).  Returns 0 or a negative EB_ERR_* code.
inline int32_t make_tmap_2d_sw128(CUtensorMap* tm, CUtensorMapDataType elem, const void* base, uint64_t rows,
                                  uint64_t row_bytes, uint64_t pitch_bytes, uint32_t box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(EB_ERR_NODEVICE, "driver entry point cuTensorMapEncodeTiled not found");
  const uint32_t esz = (elem == CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) ? 2 : 1;
  if (((uintptr_t)base & 15) || (pitch_bytes & 15) || box_rows == 0 || box_rows > 256)
    return fail(EB_ERR_ARG, "tensor map: base/pitch must be 16-byte aligned and box rows in 1..256");
  const cuuint64_t gdim[2] = {row_bytes / esz, rows};
  const cuuint64_t gstr[1] = {pitch_bytes};
  const cuuint32_t box[2] = {128 / esz, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(tm, elem, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(EB_ERR_ARG, "cuTensorMapEncodeTiled failed (%d)", (int)cr);
  return EB_OK;
}

}  // namespace eb
