// Operand layouts shared by the kernels: the 128-row x 4-column swizzled block-scale atoms
// that MXFP8 (one E8M0 per 32 K-elements) and NVFP4 (one UE4M3 per 16 K-elements) both use.
#pragma once

#include <cstddef>
#include <cstdint>

namespace mircuda_b200 {

// Byte offset of scale (row, column) in a [rows, columns] scale matrix stored as 512-byte
// atoms of 128 rows x 4 columns, atoms ordered [row_tile][column_tile], bytes inside an atom
// ordered [row % 32][row / 32 % 4][column % 4]. Same formula as the reference's
// kernels/mxfp8.cu:55-67 and sys/native/fp4_vector_sm120.cu:32-39; it is also exactly the
// 32-lane x 16-byte block that tcgen05.cp moves into tensor memory.
__host__ __device__ __forceinline__ uint32_t scale_offset(uint32_t row, uint32_t column,
                                                          uint32_t columns) {
  const uint32_t column_tiles = (columns + 3u) / 4u;
  return (((row / 128u) * column_tiles + column / 4u) * 512u) + (row % 32u) * 16u +
         ((row % 128u) / 32u) * 4u + (column % 4u);
}

// Padded size in bytes of a swizzled scale buffer (src/cutlass/mxfp8.rs:45-50 in the reference).
__host__ __device__ __forceinline__ size_t scale_bytes(size_t rows, size_t columns) {
  return ((rows + 127u) / 128u) * 128u * (((columns + 3u) / 4u) * 4u);
}

}  // namespace mircuda_b200
