// Device helpers for NVFP4 data: E2M1 code pairs -> f16x2 with the sm_100a conversion
// instruction, UE4M3 scale bytes -> fp32, and 16-byte streaming loads.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>

namespace mircuda_b200 {

__device__ __forceinline__ uint4 load_streaming_16(const void* pointer) {
  uint4 value;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
               : "l"(pointer));
  return value;
}

// Four bytes = eight E2M1 codes -> four f16x2. In every pair the low nibble (even k) lands
// in the low half.
__device__ __forceinline__ void decode_e2m1x8(uint32_t codes, __half2 (&out)[4]) {
  uint32_t r0, r1, r2, r3;
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t"
      "}\n"
      : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
      : "r"(codes));
  out[0] = *reinterpret_cast<__half2*>(&r0);
  out[1] = *reinterpret_cast<__half2*>(&r1);
  out[2] = *reinterpret_cast<__half2*>(&r2);
  out[3] = *reinterpret_cast<__half2*>(&r3);
}

// Sixteen bytes = 32 consecutive codes -> 16 f16x2 in K order.
__device__ __forceinline__ void decode_e2m1x32(const uint4& codes, __half2 (&out)[16]) {
  const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
  for (int word = 0; word < 4; ++word) {
    __half2 four[4];
    decode_e2m1x8(words[word], four);
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) out[word * 4 + pair] = four[pair];
  }
}

// UE4M3: the E4M3 bit pattern read as an unsigned value (bit 7 ignored). Every E4M3 value
// is exact in f16, so the conversion goes through the hardware e4m3x2 -> f16x2 instruction.
__device__ __forceinline__ float decode_ue4m3(uint8_t code) {
  uint32_t pair;
  const uint16_t source = static_cast<uint16_t>(code & 0x7fu);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(source));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(pair & 0xffffu)));
}

// Full E4M3 decode (sign kept, 0x7f / 0xff are NaN), through the same conversion.
__device__ __forceinline__ float decode_e4m3_signed(uint8_t code) {
  uint32_t pair;
  const uint16_t source = static_cast<uint16_t>(code);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(source));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(pair & 0xffffu)));
}

}  // namespace mircuda_b200
