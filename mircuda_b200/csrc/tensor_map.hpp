// Host-side helper that encodes TMA tensor maps. The driver entry point is looked up at run
// time through the CUDA runtime, so the library does not link against libcuda and still
// loads (for symbol checks) on a machine without a driver.
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>

namespace mircuda_b200 {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_tiled_entry() {
  static EncodeTiled entry = [] {
    void* function = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &function, cudaEnableDefault,
                                &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeTiled>(nullptr);
    }
    return reinterpret_cast<EncodeTiled>(function);
  }();
  return entry;
}

// Row-major [rows, row_bytes-wide] byte matrix, loaded as boxes of `box_rows` rows by
// 128 bytes with the 128-byte swizzle the MMA descriptors expect. `element_bytes` only
// selects the data type of the map (1 = u8, 2 = bf16/f16 as u16); extents are in elements.
inline int encode_k_major_map(CUtensorMap* map, const void* base, uint64_t rows,
                              uint64_t columns, uint32_t element_bytes, uint32_t box_rows) {
  EncodeTiled encode = encode_tiled_entry();
  if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dimensions[2] = {columns, rows};
  const cuuint64_t strides[1] = {columns * element_bytes};
  const cuuint32_t box[2] = {128u / element_bytes, box_rows};
  const cuuint32_t element_strides[2] = {1u, 1u};
  const CUtensorMapDataType type =
      element_bytes == 1u ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
  return static_cast<int>(encode(map, type, 2u, const_cast<void*>(base), dimensions, strides, box,
                                 element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
}

}  // namespace mircuda_b200
