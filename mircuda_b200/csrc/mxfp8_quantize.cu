// bf16 -> MXFP8 activation quantizer and the scale-layout conversion.
//
// Semantics follow the reference kernel `mircuda_mxfp8_quantize_bf16`
// (kernels/mxfp8.cu:69-96) bit for bit on finite inputs; the geometry does not: the
// reference runs one 32-thread block per 32-element group with 2-byte loads, this kernel
// streams 16-byte vectors (8 bf16 per thread, 4 threads per group) and writes the four
// scale bytes of an aligned group quartet as one 32-bit store into the swizzled atom.
// The kernel is bound by HBM: 2 bytes read and 1 + 1/32 bytes written per element.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "launch_overlap.hpp"
#include "layout.cuh"
#include "ptx.cuh"

namespace mircuda_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kVectorsPerThread = 4;

// Exponent byte of the block scale from the block's largest bf16 magnitude (15 bits).
// ceil(log2(amax / 448)) + 127 with 448 = 1.75 * 2^8: for amax = m * 2^e, 1 <= m < 2, this
// is e - 8 + 127, plus one when m > 1.75 (mantissa field above 0x60). Zero and subnormal
// magnitudes land on the clamp at 0, as max(amax / 448, 2^-127) does in the reference.
__device__ __forceinline__ uint32_t scale_exponent(uint32_t magnitude_bits) {
  const uint32_t exponent = magnitude_bits >> 7;
  if (exponent == 0u) return 0u;
  const int biased = static_cast<int>(exponent) - 8 + ((magnitude_bits & 0x7fu) > 0x60u ? 1 : 0);
  return static_cast<uint32_t>(max(0, min(254, biased)));
}

// 2^(127 - exponent_byte) as an fp32 (the reciprocal of the block scale); 2^-127 is the
// subnormal 0x00400000.
__device__ __forceinline__ float inverse_scale(uint32_t exponent_byte) {
  const int power = 127 - static_cast<int>(exponent_byte);
  const uint32_t bits = power >= -126 ? static_cast<uint32_t>(power + 127) << 23 : 0x00400000u;
  return __uint_as_float(bits);
}

// Largest magnitude of the eight bf16 values of a 16-byte vector, as bf16x2 (each half holds
// the maximum of its four lanes). Packed max ignores a NaN operand, as fmaxf does.
__device__ __forceinline__ uint32_t packed_abs_max(const uint4& v) {
  const __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const __nv_bfloat162 b = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  const __nv_bfloat162 c = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v.z));
  const __nv_bfloat162 d = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&v.w));
  const __nv_bfloat162 m = __hmax2(__hmax2(a, b), __hmax2(c, d));
  return *reinterpret_cast<const uint32_t*>(&m);
}

__device__ __forceinline__ uint32_t packed_max(uint32_t a, uint32_t b) {
  const __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                   *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&m);
}

// Two bf16 (packed in a u32, low half first) times `inverse` -> two E4M3 codes (low byte first).
__device__ __forceinline__ uint32_t encode_pair(uint32_t packed, float inverse) {
  const float low = __uint_as_float(packed << 16) * inverse;
  const float high = __uint_as_float(packed & 0xffff0000u) * inverse;
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp8x2(make_float2(low, high), __NV_SATFINITE, __NV_E4M3));
}

// group / groups_per_row by multiply-and-shift (group < 2^31): quotient = group * magic >> shift.
struct Divisor {
  uint32_t divisor;
  uint32_t magic;
  uint32_t shift;
};

__device__ __forceinline__ uint32_t divide(uint32_t value, const Divisor& d) {
  return static_cast<uint32_t>((static_cast<uint64_t>(value) * d.magic) >> d.shift);
}

// kBlockedInput: the [rows, columns] input is stored as column blocks one after another (block b
// holds columns b * block_columns .. of every row as a contiguous [rows, block_columns] matrix:
// the rank-major layout an all-gather of column shards produces); `block_row_vectors` and
// `block_vectors` are block_columns / 8 and rows * block_columns / 8. Outputs are the same as for
// the row-major input.
template <bool kPackedScales, bool kBlockedInput = false>
__global__ void __launch_bounds__(kThreads)
mxfp8_quantize_kernel(const uint4* __restrict__ input, uint2* __restrict__ output,
                      uint8_t* __restrict__ scales, uint32_t vectors, Divisor groups_per_row,
                      uint32_t block_row_vectors = 0u, uint32_t block_vectors = 0u) {
  const uint32_t first = blockIdx.x * (kThreads * kVectorsPerThread) + threadIdx.x;
  // The consumer of the codes (normally the GEMM) may set itself up while this grid runs;
  // this grid waits for everything before it on the stream before its first access.
  ptx::dependency_launch_next();
  ptx::dependency_wait();

  uint4 values[kVectorsPerThread];
#pragma unroll
  for (int item = 0; item < kVectorsPerThread; ++item) {
    const uint32_t vector = first + item * kThreads;
    uint32_t source = vector;
    if constexpr (kBlockedInput) {
      const uint32_t row = divide(vector / 4u, groups_per_row);
      const uint32_t column_vector = vector - row * (groups_per_row.divisor * 4u);
      const uint32_t block = column_vector / block_row_vectors;
      source = block * block_vectors + row * block_row_vectors + (column_vector - block * block_row_vectors);
    }
    values[item] = vector < vectors ? __ldg(input + source) : make_uint4(0u, 0u, 0u, 0u);
  }

#pragma unroll
  for (int item = 0; item < kVectorsPerThread; ++item) {
    const uint32_t vector = first + item * kThreads;
    const uint4 v = values[item];
    uint32_t both = packed_abs_max(v);
    both = packed_max(both, __shfl_xor_sync(0xffffffffu, both, 1));
    both = packed_max(both, __shfl_xor_sync(0xffffffffu, both, 2));
    uint32_t maximum = max(both & 0xffffu, both >> 16);
    if (maximum > 0x7f80u) maximum = 0u;  // only when every element of the block is NaN
    const uint32_t exponent = scale_exponent(maximum);
    const float inverse = inverse_scale(exponent);
    const uint32_t low = encode_pair(v.x, inverse) | (encode_pair(v.y, inverse) << 16);
    const uint32_t high = encode_pair(v.z, inverse) | (encode_pair(v.w, inverse) << 16);
    if (vector < vectors) output[vector] = make_uint2(low, high);

    // One scale byte per 4-thread group. A warp holds 8 consecutive groups; when rows are a
    // multiple of 128 columns those are two aligned quartets whose bytes are adjacent in the
    // swizzled atom, so lanes 0 and 16 each write one 32-bit word.
    if constexpr (kPackedScales) {
      const uint32_t lane = threadIdx.x & 31u;
      const uint32_t base = lane & 16u;
      const uint32_t word = __shfl_sync(0xffffffffu, exponent, base) |
                            (__shfl_sync(0xffffffffu, exponent, base + 4u) << 8) |
                            (__shfl_sync(0xffffffffu, exponent, base + 8u) << 16) |
                            (__shfl_sync(0xffffffffu, exponent, base + 12u) << 24);
      if ((lane & 15u) == 0u && vector < vectors) {
        const uint32_t group = vector / 4u;
        const uint32_t row = divide(group, groups_per_row);
        const uint32_t group_in_row = group - row * groups_per_row.divisor;
        *reinterpret_cast<uint32_t*>(
            scales + scale_offset(row, group_in_row, groups_per_row.divisor)) = word;
      }
    } else {
      if ((threadIdx.x & 3u) == 0u && vector < vectors) {
        const uint32_t group = vector / 4u;
        const uint32_t row = divide(group, groups_per_row);
        const uint32_t group_in_row = group - row * groups_per_row.divisor;
        scales[scale_offset(row, group_in_row, groups_per_row.divisor)] =
            static_cast<uint8_t>(exponent);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
mxfp8_swizzle_scales_kernel(const uint8_t* __restrict__ input, uint8_t* __restrict__ output,
                      uint32_t rows, uint32_t columns) {
  const uint64_t index = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= static_cast<uint64_t>(rows) * columns) return;
  const uint32_t row = static_cast<uint32_t>(index / columns);
  const uint32_t column = static_cast<uint32_t>(index % columns);
  output[scale_offset(row, column, columns)] = input[index];
}

}  // namespace
}  // namespace mircuda_b200

namespace mircuda_b200 {
namespace {

// block_columns == 0: row-major input.
int launch_mxfp8_quantize(const void* input, void* output, void* scales, uint32_t rows, uint32_t columns,
                          uint32_t block_columns, void* stream) {
  if (input == nullptr || output == nullptr || scales == nullptr || stream == nullptr ||
      rows == 0u || columns == 0u || columns % 32u != 0u) {
    return -1;
  }
  if (block_columns != 0u && (block_columns % 8u != 0u || columns % block_columns != 0u)) return -1;
  if ((reinterpret_cast<uintptr_t>(input) & 15u) != 0u ||
      (reinterpret_cast<uintptr_t>(output) & 7u) != 0u ||
      (reinterpret_cast<uintptr_t>(scales) & 3u) != 0u) {
    return -1;
  }
  const uint64_t vectors = static_cast<uint64_t>(rows) * (columns / 8u);
  if (vectors >= (1ull << 32)) return -1;  // group indices are 32-bit inside the kernel
  const uint64_t per_block = kThreads * kVectorsPerThread;
  const uint64_t blocks = (vectors + per_block - 1u) / per_block;
  // Exact multiply-and-shift division for dividends below 2^31: with s = ceil(log2(d)) and
  // magic = ceil(2^(31+s) / d) < 2^32, floor(n / d) == (n * magic) >> (31 + s).
  Divisor divisor{columns / 32u, 0u, 0u};
  uint32_t log2_ceiling = 0;
  while ((1ull << log2_ceiling) < divisor.divisor) ++log2_ceiling;
  divisor.shift = 31u + log2_ceiling;
  divisor.magic = static_cast<uint32_t>(((1ull << divisor.shift) + divisor.divisor - 1u) /
                                        divisor.divisor);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned int>(blocks), 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = overlap_launches() ? 1u : 0u;
  const bool packed = columns % 128u == 0u;
  const bool blocked = block_columns != 0u && block_columns != columns;
  auto function = blocked ? (packed ? mxfp8_quantize_kernel<true, true> : mxfp8_quantize_kernel<false, true>)
                          : (packed ? mxfp8_quantize_kernel<true, false> : mxfp8_quantize_kernel<false, false>);
  const uint32_t block_row_vectors = blocked ? block_columns / 8u : 0u;
  const uint32_t block_vectors = blocked ? rows * (block_columns / 8u) : 0u;
  return static_cast<int>(cudaLaunchKernelEx(
      &config, function, static_cast<const uint4*>(input), static_cast<uint2*>(output),
      static_cast<uint8_t*>(scales), static_cast<uint32_t>(vectors), divisor, block_row_vectors, block_vectors));
}

}  // namespace
}  // namespace mircuda_b200

extern "C" int mircuda_b200_mxfp8_quantize_bf16(const void* input, void* output, void* scales,
                                                uint32_t rows, uint32_t columns, void* stream) {
  return mircuda_b200::launch_mxfp8_quantize(input, output, scales, rows, columns, 0u, stream);
}

extern "C" int mircuda_b200_mxfp8_quantize_bf16_blocks(const void* input, void* output, void* scales,
                                                       uint32_t rows, uint32_t columns,
                                                       uint32_t block_columns, void* stream) {
  if (block_columns == 0u) return -1;
  return mircuda_b200::launch_mxfp8_quantize(input, output, scales, rows, columns, block_columns, stream);
}

extern "C" int mircuda_b200_mxfp8_swizzle_scales(const void* input, void* output, uint32_t rows,
                                                 uint32_t columns, void* stream) {
  using namespace mircuda_b200;
  if (input == nullptr || output == nullptr || stream == nullptr || rows == 0u || columns == 0u) {
    return -1;
  }
  const uint64_t elements = static_cast<uint64_t>(rows) * columns;
  const uint64_t blocks = (elements + 255u) / 256u;
  if (blocks > 0x7fffffffull) return -1;
  mxfp8_swizzle_scales_kernel<<<static_cast<unsigned int>(blocks), 256, 0,
                          static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(input), static_cast<uint8_t*>(output), rows, columns);
  return static_cast<int>(cudaPeekAtLastError());
}
