// Host-side construction of TMA tensor maps through the driver entry point (no link-time
// dependency on libcuda, so the library also loads on a machine without a driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace eredu {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] with `ld` elements between rows; box = [box_rows, box_cols]
// (box_cols * elem_bytes must be 128 for SWIZZLE_128B). Out-of-range elements read as zero.
// Returns 0 on success.
inline int make_tma_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                       uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                       CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld * elem_bytes) & 15) != 0) return -2;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 3-D tensor [d2, d1, d0] (d0 innermost) with byte strides for d1 and d2; box = [b2, b1, b0].
inline int make_tma_3d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t d0,
                       uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0,
                       uint32_t b1, uint32_t b2, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (stride1_bytes & 15) != 0 || (stride2_bytes & 15) != 0)
    return -2;
  cuuint64_t gdim[3] = {d0, d1, d2};
  cuuint64_t gstride[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  (void)elem_bytes;
  CUresult r = fn(map, dtype, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 4-D tensor [d3, d2, d1, d0] (d0 innermost) with byte strides for d1..d3; box = [b3, b2, b1, b0].
inline int make_tma_4d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, uint64_t d0, uint64_t d1, uint64_t d2,
                       uint64_t d3, uint64_t stride1_bytes, uint64_t stride2_bytes, uint64_t stride3_bytes, uint32_t b0,
                       uint32_t b1, uint32_t b2, uint32_t b3, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (stride1_bytes & 15) != 0 || (stride2_bytes & 15) != 0 ||
      (stride3_bytes & 15) != 0)
    return -2;
  cuuint64_t gdim[4] = {d0, d1, d2, d3};
  cuuint64_t gstride[3] = {stride1_bytes, stride2_bytes, stride3_bytes};
  cuuint32_t box[4] = {b0, b1, b2, b3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, dtype, 4, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace eredu
