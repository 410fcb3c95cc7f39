// bf16 -> NVFP4 quantizer (E2M1 codes, one UE4M3 scale per 16 K-elements, per-tensor fp32
// global scale). The reference has no such quantizer; the rule implemented here is
//   global = amax_tensor / (448 * 6)              (1.0 for an all-zero tensor)
//   s_blk  = rne_ue4m3(amax_blk / (6 * global))
//   code   = rne_e2m1(x / (ue4m3(s_blk) * global)), saturating at +-6; 0 when s_blk == 0
// with every operation in round-to-nearest fp32. Conversions use the sm_100a cvt
// instructions. The kernel is bound by HBM: 2 bytes in, 0.5625 bytes out per element.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "fp4_codec.cuh"
#include "layout.cuh"

namespace mircuda_b200 {
namespace {

__device__ __forceinline__ uint32_t magnitude_bits(uint32_t half_bits) {
  const uint32_t magnitude = half_bits & 0x7fffu;
  return magnitude > 0x7f80u ? 0u : magnitude;  // NaN takes no part in amax
}

__device__ __forceinline__ uint32_t max_magnitude(const uint4& v) {
  uint32_t result = max(max(magnitude_bits(v.x), magnitude_bits(v.x >> 16)),
                        max(magnitude_bits(v.y), magnitude_bits(v.y >> 16)));
  return max(result, max(max(magnitude_bits(v.z), magnitude_bits(v.z >> 16)),
                         max(magnitude_bits(v.w), magnitude_bits(v.w >> 16))));
}

// Largest |x| as bf16 magnitude bits, combined across the grid with an integer atomic max.
__global__ void __launch_bounds__(256)
nvfp4_amax_kernel(const uint4* __restrict__ input, size_t vectors, const uint16_t* __restrict__ tail,
            size_t tail_elements, unsigned int* __restrict__ result) {
  uint32_t maximum = 0u;
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < vectors;
       index += static_cast<size_t>(gridDim.x) * blockDim.x) {
    maximum = max(maximum, max_magnitude(__ldg(input + index)));
  }
  if (blockIdx.x == 0 && threadIdx.x < tail_elements) {
    maximum = max(maximum, magnitude_bits(tail[threadIdx.x]));
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    maximum = max(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
  }
  if ((threadIdx.x & 31) == 0 && maximum != 0u) atomicMax(result, maximum);
}

__global__ void nvfp4_finish_global_scale_kernel(unsigned int* word) {
  const uint32_t magnitude = *word;  // bf16 bits of the tensor amax
  const float amax = __uint_as_float(magnitude << 16);
  const float global = amax > 0.0f ? __fdiv_rn(amax, 2688.0f) : 1.0f;
  *reinterpret_cast<float*>(word) = global;
}

__device__ __forceinline__ uint32_t encode_e2m1_pair(float low, float high) {
  uint16_t packed;
  asm("{\n\t"
      ".reg .b8 byte;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 byte, %2, %1;\n\t"
      "cvt.u16.u8 %0, byte;\n\t"
      "}\n"
      : "=h"(packed)
      : "f"(low), "f"(high));
  return packed;
}

// One thread per 16-element block: two 16-byte loads, one 8-byte store, one scale byte.
// ROW_MAJOR_SCALES: scales go to [rows, k/16] bytes instead of the swizzled atoms, so that
// whole rows (codes and scales) can be moved to another place before the layout is fixed.
// SwiGLU of eight (gate, up) bf16 pairs -> eight bf16, as the stand-alone SwiGLU kernel
// computes and rounds them.
__device__ __forceinline__ uint4 swiglu8(const uint4& gate, const uint4& up) {
  const uint32_t gates[4] = {gate.x, gate.y, gate.z, gate.w};
  const uint32_t ups[4] = {up.x, up.y, up.z, up.w};
  uint32_t packed[4];
#pragma unroll
  for (int word = 0; word < 4; ++word) {
    const float g_low = __uint_as_float(gates[word] << 16);
    const float g_high = __uint_as_float(gates[word] & 0xffff0000u);
    const float u_low = __uint_as_float(ups[word] << 16);
    const float u_high = __uint_as_float(ups[word] & 0xffff0000u);
    const __nv_bfloat162 two = __floats2bfloat162_rn(
        __fdividef(g_low, 1.0f + __expf(-g_low)) * u_low,
        __fdividef(g_high, 1.0f + __expf(-g_high)) * u_high);
    packed[word] = *reinterpret_cast<const uint32_t*>(&two);
  }
  return make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// SWIGLU: the input is [rows, 2k] (gate columns then up columns) and the quantised tensor is
// silu(gate) * up rounded to bf16, which is never written to memory.
template <bool ROW_MAJOR_SCALES, bool SWIGLU>
__global__ void __launch_bounds__(256)
nvfp4_quantize_kernel(const uint4* __restrict__ input, const float* __restrict__ global_scale,
                uint2* __restrict__ codes, uint8_t* __restrict__ scales, uint32_t rows,
                const unsigned int* __restrict__ row_bound, uint32_t k) {
  if (row_bound != nullptr) rows = min(rows, __ldg(row_bound));
  const uint32_t blocks_per_row = k / 16u;
  const size_t block = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (block >= static_cast<size_t>(rows) * blocks_per_row) return;
  uint4 first, second;
  if (SWIGLU) {
    const size_t row_index = block / blocks_per_row;
    const size_t vector = row_index * (blocks_per_row * 4u) + (block - row_index * blocks_per_row) * 2u;
    const size_t up = vector + blocks_per_row * 2u;       // k / 8 sixteen-byte vectors further
    first = swiglu8(__ldg(input + vector), __ldg(input + up));
    second = swiglu8(__ldg(input + vector + 1u), __ldg(input + up + 1u));
  } else {
    first = __ldg(input + block * 2u);
    second = __ldg(input + block * 2u + 1u);
  }
  const float global = *global_scale;
  const uint32_t magnitude = max(max_magnitude(first), max_magnitude(second));
  const float block_max = __uint_as_float(magnitude << 16);
  const float requested = __fdiv_rn(block_max, __fmul_rn(6.0f, global));
  uint8_t scale_code = 0u;
  if (requested > 0.0f) {
    scale_code = static_cast<uint8_t>(
        __nv_cvt_float_to_fp8(requested, __NV_SATFINITE, __NV_E4M3) & 0x7fu);
  }
  const float denominator = __fmul_rn(decode_ue4m3(scale_code), global);
  const uint32_t words[8] = {first.x, first.y, first.z, first.w,
                             second.x, second.y, second.z, second.w};
  uint32_t out[2] = {0u, 0u};
  // One correctly rounded reciprocal per block, then exact-rounded products: 16 divisions
  // fewer per block (they made this memory-bound kernel arithmetic-bound). Where the
  // reciprocal overflows (tensors whose largest magnitude is below about 1e-30) the block
  // divides instead, as the written definition says.
  const float inverse = __frcp_rn(denominator);
  if (scale_code != 0u && inverse <= 3.402823466e38f) {
#pragma unroll
    for (int word = 0; word < 8; ++word) {
      const float low = __fmul_rn(__uint_as_float(words[word] << 16), inverse);
      const float high = __fmul_rn(__uint_as_float(words[word] & 0xffff0000u), inverse);
      out[word / 4] |= encode_e2m1_pair(low, high) << ((word % 4) * 8);
    }
  } else if (scale_code != 0u) {
#pragma unroll
    for (int word = 0; word < 8; ++word) {
      const float low = __fdiv_rn(__uint_as_float(words[word] << 16), denominator);
      const float high = __fdiv_rn(__uint_as_float(words[word] & 0xffff0000u), denominator);
      out[word / 4] |= encode_e2m1_pair(low, high) << ((word % 4) * 8);
    }
  }
  codes[block] = make_uint2(out[0], out[1]);
  const uint32_t row = static_cast<uint32_t>(block / blocks_per_row);
  const uint32_t column = static_cast<uint32_t>(block % blocks_per_row);
  scales[ROW_MAJOR_SCALES ? block : scale_offset(row, column, blocks_per_row)] = scale_code;
}

}  // namespace
}  // namespace mircuda_b200

extern "C" int mircuda_b200_nvfp4_global_scale(const void* input, size_t elements,
                                               void* global_scale, void* stream) {
  using namespace mircuda_b200;
  if (input == nullptr || global_scale == nullptr || stream == nullptr || elements == 0u) return -1;
  if ((reinterpret_cast<uintptr_t>(input) & 15u) != 0u ||
      (reinterpret_cast<uintptr_t>(global_scale) & 3u) != 0u) {
    return -1;
  }
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  int status = static_cast<int>(cudaMemsetAsync(global_scale, 0, sizeof(float), cuda_stream));
  if (status != 0) return status;
  const size_t vectors = elements / 8u;
  const size_t tail = elements % 8u;
  size_t blocks = (vectors + 255u) / 256u;
  if (blocks > 148u * 8u) blocks = 148u * 8u;
  if (blocks == 0u) blocks = 1u;
  nvfp4_amax_kernel<<<static_cast<unsigned int>(blocks), 256, 0, cuda_stream>>>(
      static_cast<const uint4*>(input), vectors,
      static_cast<const uint16_t*>(input) + vectors * 8u, tail,
      static_cast<unsigned int*>(global_scale));
  nvfp4_finish_global_scale_kernel<<<1, 1, 0, cuda_stream>>>(static_cast<unsigned int*>(global_scale));
  return static_cast<int>(cudaPeekAtLastError());
}

namespace mircuda_b200 {
namespace {

template <bool ROW_MAJOR_SCALES, bool SWIGLU = false>
int launch_quantize(const void* input, const void* global_scale, void* codes, void* scales,
                    uint32_t rows, uint32_t k, void* stream,
                    const unsigned int* row_bound = nullptr) {
  if (input == nullptr || global_scale == nullptr || codes == nullptr || scales == nullptr ||
      stream == nullptr || rows == 0u || k == 0u || k % 64u != 0u) {
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(input) & 15u) != 0u ||
      (reinterpret_cast<uintptr_t>(codes) & 7u) != 0u) {
    return -1;
  }
  const size_t blocks = static_cast<size_t>(rows) * (k / 16u);
  const size_t grid = (blocks + 255u) / 256u;
  if (grid > 0x7fffffffull) return -1;
  nvfp4_quantize_kernel<ROW_MAJOR_SCALES, SWIGLU>
      <<<static_cast<unsigned int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
          static_cast<const uint4*>(input), static_cast<const float*>(global_scale),
          static_cast<uint2*>(codes), static_cast<uint8_t*>(scales), rows, row_bound, k);
  return static_cast<int>(cudaPeekAtLastError());
}

}  // namespace
}  // namespace mircuda_b200

extern "C" int mircuda_b200_nvfp4_quantize_bf16(const void* input, const void* global_scale,
                                                void* codes, void* scales, uint32_t rows,
                                                uint32_t k, void* stream) {
  return mircuda_b200::launch_quantize<false>(input, global_scale, codes, scales, rows, k, stream);
}

extern "C" int mircuda_b200_nvfp4_quantize_rows_bf16(const void* input, const void* global_scale,
                                                     void* codes, void* row_scales, uint32_t rows,
                                                     uint32_t k, void* stream) {
  return mircuda_b200::launch_quantize<true>(input, global_scale, codes, row_scales, rows, k, stream);
}

extern "C" int mircuda_b200_moe_swiglu_nvfp4(const void* input, const void* global_scale,
                                             void* codes, void* scales, uint32_t rows,
                                             const unsigned int* row_bound, uint32_t intermediate,
                                             void* stream) {
  return mircuda_b200::launch_quantize<false, true>(input, global_scale, codes, scales, rows,
                                                    intermediate, stream, row_bound);
}
