// Host-side construction of TMA tensor maps without linking libcuda directly:
// the encoder is looked up through the runtime's driver entry point query.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

namespace b200 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
      throw std::runtime_error("cuTensorMapEncodeTiled is not available from the installed driver");
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// The encoder is a driver entry point and needs the device's context current on the calling thread. A thread that has
// made no runtime call yet (an autograd worker whose first operation is a GEMM on device 0: the device guard sees
// "already device 0" and calls nothing) has none, and the encoder answers CUDA_ERROR_INVALID_CONTEXT. Binding the primary
// context with a harmless runtime call and encoding again fixes that; the normal path pays nothing.
inline CUresult encode_tiled(CUtensorMap* m, CUtensorMapDataType type, cuuint32_t rank, void* base, const cuuint64_t* dims,
                             const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* estr, CUtensorMapSwizzle swizzle) {
  CUresult r = tensor_map_encoder()(m, type, rank, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
    cudaFree(nullptr);
    r = tensor_map_encoder()(m, type, rank, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r;
}

// 2-D tensor map over a row-major matrix of 16-bit elements.
//   inner      : number of contiguous elements per row
//   outer      : number of rows
//   row_stride : elements between consecutive rows (multiple of 8)
//   box_inner / box_outer : tile fetched per copy (box_inner * 2 bytes <= 128 when swizzled)
inline CUtensorMap make_tensor_map_2d_b16(const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride,
                                          uint32_t box_inner, uint32_t box_outer, bool swizzle128 = true) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((row_stride * 2) % 16 != 0) throw std::runtime_error("TMA row stride must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_tiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return m;
}

// 2-D tensor map over a row-major matrix of bytes (8-bit floats): strides and boxes in bytes = elements.
inline CUtensorMap make_tensor_map_2d_u8(const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride, uint32_t box_inner,
                                         uint32_t box_outer) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if (row_stride % 16 != 0) throw std::runtime_error("TMA row stride must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_tiled(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled (u8) failed with code " + std::to_string(int(r)));
  return m;
}

// 2-D tensor map over a row-major fp32 matrix (sizes and stride in elements; box_inner * 4 bytes <= 128 when swizzled).
inline CUtensorMap make_tensor_map_2d_f32(const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride, uint32_t box_inner,
                                          uint32_t box_outer, bool swizzle128 = true) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((row_stride * 4) % 16 != 0) throw std::runtime_error("TMA row stride must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride * 4};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_tiled(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled (f32) failed with code " + std::to_string(int(r)));
  return m;
}

// 3-D variant: [outer2][outer][inner] with explicit strides (elements) for the two outer dims.
inline CUtensorMap make_tensor_map_3d_b16(const void* base, uint64_t inner, uint64_t outer, uint64_t outer2,
                                          uint64_t stride_outer, uint64_t stride_outer2, uint32_t box_inner,
                                          uint32_t box_outer, uint32_t box_outer2, bool swizzle128 = true) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((stride_outer * 2) % 16 != 0 || (stride_outer2 * 2) % 16 != 0)
    throw std::runtime_error("TMA strides must be multiples of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[3] = {inner, outer, outer2};
  cuuint64_t strides[2] = {stride_outer * 2, stride_outer2 * 2};
  cuuint32_t box[3] = {box_inner, box_outer, box_outer2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_tiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return m;
}

}  // namespace b200
