// Weight-only MXFP8 projection: out[t, n] = bf16(sum_k x[t, k] * e4m3(w[n, k]) * 2^(s[n, k/32] - 127))
// with bf16 activations that are NOT quantised, E4M3 weights handed over as little-endian
// u32 words and row-major [N, K/32] E8M0 scales. Replaces the reference's run-time-compiled
// kernels `mircuda_mxfp8_bf16` / `mircuda_mxfp8_bf16_tiled` (kernels/mxfp8.cu:111-217) and
// their launches (src/mxfp8/matmul.rs:131-157).
//
// For decode-sized token counts the op is bound by streaming the weights (N*K bytes). One
// warp owns one output row and up to four tokens; each lane reads 16 weight bytes per step
// with a streaming 16-byte load (the reference reads single bytes), decodes them with the
// hardware e4m3x2 -> f16x2 conversion (exact) and accumulates in fp32, applying the block
// scale once per 16 products.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "fp4_codec.cuh"

namespace mircuda_b200 {
namespace {

constexpr int kWarps = 8;
constexpr int kTokenTile = 4;

__device__ __forceinline__ float2 decode_e4m3x2(uint32_t two_codes) {
  uint32_t pair;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(static_cast<uint16_t>(two_codes)));
  return __half22float2(*reinterpret_cast<const __half2*>(&pair));
}

__global__ void __launch_bounds__(kWarps * 32)
mxfp8_weight_only_kernel(const __nv_bfloat16* __restrict__ input, const uint8_t* __restrict__ weight,
                   const uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ output,
                   uint32_t tokens, uint32_t k, uint32_t n) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  const uint32_t token0 = blockIdx.y * kTokenTile;
  if (row >= n) return;
  const uint32_t groups = k / 32u;
  float sums[kTokenTile] = {};

  if ((k & 15u) == 0u && (reinterpret_cast<uintptr_t>(weight) & 15u) == 0u &&
      (reinterpret_cast<uintptr_t>(input) & 15u) == 0u) {
    const uint8_t* weight_row = weight + static_cast<size_t>(row) * k;
    for (uint32_t column = lane * 16u; column < k; column += 512u) {
      const uint4 packed = load_streaming_16(weight_row + column);
      const uint32_t exponent = scales[static_cast<size_t>(row) * groups + column / 32u];
      const float block_scale =  // 2^(e-127); 2^-127 is the subnormal 0x00400000
          exponent == 0u ? 5.87747175e-39f : __uint_as_float(exponent << 23);
      const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
      float w[16];
#pragma unroll
      for (int word = 0; word < 4; ++word) {
        const float2 low = decode_e4m3x2(words[word] & 0xffffu);
        const float2 high = decode_e4m3x2(words[word] >> 16);
        w[word * 4 + 0] = low.x;
        w[word * 4 + 1] = low.y;
        w[word * 4 + 2] = high.x;
        w[word * 4 + 3] = high.y;
      }
#pragma unroll
      for (int item = 0; item < kTokenTile; ++item) {
        const uint32_t token = token0 + item;
        if (token < tokens) {
          const uint4* x = reinterpret_cast<const uint4*>(input + static_cast<size_t>(token) * k + column);
          const uint4 first = __ldg(x);
          const uint4 second = __ldg(x + 1);
          const uint32_t xs[8] = {first.x, first.y, first.z, first.w,
                                  second.x, second.y, second.z, second.w};
          float partial = 0.0f;
#pragma unroll
          for (int pair = 0; pair < 8; ++pair) {
            partial = fmaf(__uint_as_float(xs[pair] << 16), w[pair * 2], partial);
            partial = fmaf(__uint_as_float(xs[pair] & 0xffff0000u), w[pair * 2 + 1], partial);
          }
          sums[item] = fmaf(partial, block_scale, sums[item]);
        }
      }
    }
  } else {
    for (uint32_t column = lane; column < k; column += 32u) {
      const uint8_t code = weight[static_cast<size_t>(row) * k + column];
      const uint8_t exponent = scales[static_cast<size_t>(row) * groups + column / 32u];
      const float scale = exponent == 0u ? 5.87747175e-39f
                                         : __uint_as_float(static_cast<uint32_t>(exponent) << 23);
      const float w = decode_e4m3x2(code).x * scale;
#pragma unroll
      for (int item = 0; item < kTokenTile; ++item) {
        const uint32_t token = token0 + item;
        if (token < tokens) {
          sums[item] = fmaf(__bfloat162float(input[static_cast<size_t>(token) * k + column]), w,
                            sums[item]);
        }
      }
    }
  }

#pragma unroll
  for (int item = 0; item < kTokenTile; ++item) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      sums[item] += __shfl_xor_sync(0xffffffffu, sums[item], offset);
    }
    const uint32_t token = token0 + item;
    if (lane == 0u && token < tokens) {
      output[static_cast<size_t>(token) * n + row] = __float2bfloat16_rn(sums[item]);
    }
  }
}

}  // namespace
}  // namespace mircuda_b200

extern "C" int mircuda_b200_mxfp8_bf16(const void* input, const void* weight, const void* scales,
                                       void* output, uint32_t tokens, uint32_t input_features,
                                       uint32_t output_features, void* stream) {
  using namespace mircuda_b200;
  if (input == nullptr || weight == nullptr || scales == nullptr || output == nullptr ||
      stream == nullptr || tokens == 0u || input_features == 0u || output_features == 0u ||
      input_features % 32u != 0u) {
    return -1;
  }
  const dim3 grid((output_features + kWarps - 1) / kWarps, (tokens + kTokenTile - 1) / kTokenTile);
  if (grid.y > 65535u) return -1;
  mxfp8_weight_only_kernel<<<grid, kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
      static_cast<const uint8_t*>(scales), static_cast<__nv_bfloat16*>(output), tokens,
      input_features, output_features);
  return static_cast<int>(cudaPeekAtLastError());
}
