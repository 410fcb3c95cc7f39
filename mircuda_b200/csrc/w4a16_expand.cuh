// Device helpers shared by the fused int4 W4A16 GEMM kernels (w4a16_tile.cu, w4a16_pair.cu): the
// expansion of eight packed codes to f16 and the shared-memory accesses of the converter warps.
#pragma once

#include <cstdint>

namespace mircuda_b200 {
namespace w4a16_expand {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Eight codes of one word (k ascending from the low nibble) -> (q - 8) * scale as four f16x2 in
// K order. 0x6400 is 1024.0 in f16: OR-ing a nibble into its mantissa gives 1024 + q exactly.
__device__ __forceinline__ uint4 expand8(uint32_t codes, uint32_t scale2) {
  constexpr uint32_t kMask = 0x000f000fu, kMagic = 0x64006400u, kBias = 0x64086408u;   // 1032.0
  const uint32_t v04 = mul_f16x2(sub_f16x2((codes & kMask) | kMagic, kBias), scale2);           // k0, k4
  const uint32_t v15 = mul_f16x2(sub_f16x2(((codes >> 4) & kMask) | kMagic, kBias), scale2);    // k1, k5
  const uint32_t v26 = mul_f16x2(sub_f16x2(((codes >> 8) & kMask) | kMagic, kBias), scale2);    // k2, k6
  const uint32_t v37 = mul_f16x2(sub_f16x2(((codes >> 12) & kMask) | kMagic, kBias), scale2);   // k3, k7
  return make_uint4(prmt(v04, v15, 0x5410u), prmt(v26, v37, 0x5410u), prmt(v04, v15, 0x7632u),
                    prmt(v26, v37, 0x7632u));
}

__device__ __forceinline__ uint4 load_shared_16(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(address)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t load_shared_u16(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(address) : "memory");
  return v;
}

__device__ __forceinline__ void store_shared_u16(uint32_t address, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(address), "h"(static_cast<uint16_t>(v)) : "memory");
}

__device__ __forceinline__ void store_shared_16(uint32_t address, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

}  // namespace w4a16_expand
}  // namespace mircuda_b200
