// Host-side TMA descriptor encoding. The driver entry point is resolved at run
// time through the CUDA runtime, so the library links against libcudart only and
// loads on machines without a driver (build check on CPU-only boxes).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace mbh {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, inner] with `row_bytes` pitch; box = [box_rows, box_inner];
// 128-byte swizzle (box_inner * elem size must be 128 bytes), zero fill out of bounds.
inline int encode_2d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t inner,
                     uint64_t rows, uint64_t row_bytes, uint32_t box_inner, uint32_t box_rows,
                     CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -4;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_bytes & 15)) return -1;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

// 3-D tensor [d2, d1, inner] with byte strides s1 (between d1 rows) and s2.
inline int encode_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t inner,
                     uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t box_inner,
                     uint32_t box1, uint32_t box2,
                     CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -4;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1 & 15) || (s2 & 15)) return -1;
  cuuint64_t dims[3] = {inner, d1, d2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {box_inner, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

}  // namespace mbh
