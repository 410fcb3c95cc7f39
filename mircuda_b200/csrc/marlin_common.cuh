// Device helpers shared by the Marlin-layout W4A16 kernels (dense and MoE): E2M1 bit placement
// into bf16, the prepared-scale multiplier and the bf16 mma.sync wrapper.
#pragma once

#include <cstdint>

namespace mircuda_b200 {
namespace marlin {

__device__ __forceinline__ void place_e2m1x8(uint32_t q, uint32_t (&out)[4]) {
  out[3] = (q & 0x80008000u) | ((q & 0x70007000u) >> 6);
  q <<= 4;
  out[2] = (q & 0x80008000u) | ((q & 0x70007000u) >> 6);
  q <<= 4;
  out[1] = (q & 0x80008000u) | ((q & 0x70007000u) >> 6);
  q <<= 4;
  out[0] = (q & 0x80008000u) | ((q & 0x70007000u) >> 6);
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1,
                                                 uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Prepared scale byte c = upper 8 bits (without sign) of the f16 v = s * factor * 128, or 0.
// Returns v * 2^110 as a bf16 in both halves: exponent field (c >> 3) - 15 + 127 + 110, top
// three mantissa bits c & 7, i.e. (c + 1776) << 4.
__device__ __forceinline__ uint32_t scale_multiplier(uint32_t code) {
  const uint32_t bits = code == 0u ? 0u : (code + 1776u) << 4;
  return bits | (bits << 16);
}

}  // namespace marlin
}  // namespace mircuda_b200
