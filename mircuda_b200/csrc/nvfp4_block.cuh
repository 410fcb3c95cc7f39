// Device helpers shared by the NVFP4 quantizer kernels and by epilogues that quantise what they
// have just computed: one 16-element block of bf16 values -> eight code bytes and one UE4M3
// scale byte, for a given tensor (global) scale; SwiGLU of bf16 pairs as the stand-alone
// kernel computes and rounds it. The rule (no reference counterpart exists) is
//   s_blk = rne_ue4m3(amax_blk / (6 * global))
//   code  = rne_e2m1(x * r), r = fl32(1 / (ue4m3(s_blk) * global)) taken once per block
//           (x / (ue4m3(s_blk) * global) where r overflows), saturating at +-6; 0 when s_blk == 0
// with every operation in round-to-nearest fp32 and the sm_100a conversion instructions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <cstdint>

#include "fp4_codec.cuh"

namespace mircuda_b200 {
namespace nvfp4_block {

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

// Sixteen bf16 values (`first` = elements 0..7, `second` = 8..15, two per word, even element
// low) -> eight code bytes (even element in the low nibble) and the block's scale byte.
__device__ __forceinline__ uint2 quantize_block16(const uint4& first, const uint4& second, float global,
                                                  uint8_t* scale_out) {
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
  // fewer per block (they made the memory-bound quantizer arithmetic-bound). Where the
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
  *scale_out = scale_code;
  return make_uint2(out[0], out[1]);
}

}  // namespace nvfp4_block
}  // namespace mircuda_b200
