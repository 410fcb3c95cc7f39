// Blockwise-scaled FP8 GEMV, M = 1: y[n] = bf16(sum_b sa[b] * sb[n / 128, b] * sum_{k in block b}
// e4m3(x[k]) * e4m3(W[n, k])) with 128-element K blocks, fp32 scales (one per block of the
// input, one per 128 x 128 block of the weights) and fp32 accumulation. Replaces the
// reference's CUTLASS Sm120 blockwise kernel (sys/native/fp8_vector_sm120.cu:92-142) behind
// the same C entry points; n and k are multiples of 128 as there. The weight scales are read
// in CUTLASS's default MN-major order, index n / 128 + b * (n / 128): the reference's only
// test is constant-valued, so this order is not pinned by it.
//
// The op streams N*K bytes once and is bound by HBM: one warp per output row, 16 weight bytes
// per lane and step with a streaming 16-byte load, hardware e4m3x2 -> f16x2 decoding (exact),
// products accumulated in fp32 per 128-block and scaled once per block.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <new>

#include "fp4_codec.cuh"

namespace mircuda_b200 {
namespace fp8_vector {

constexpr int kWarps = 8;

struct Plan {
  int n, k;
  cudaStream_t stream;
};

__device__ __forceinline__ float2 decode_pair(uint32_t two_codes) {
  uint32_t pair;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(static_cast<uint16_t>(two_codes)));
  return __half22float2(*reinterpret_cast<const __half2*>(&pair));
}

__global__ void __launch_bounds__(kWarps * 32)
fp8_vector_kernel(const uint8_t* __restrict__ input, const float* __restrict__ input_scales,
                  const uint8_t* __restrict__ weight, const float* __restrict__ weight_scales,
                  __nv_bfloat16* __restrict__ output, uint32_t n, uint32_t k) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= n) return;
  const uint32_t blocks_n = n / 128u;
  const uint8_t* weight_row = weight + static_cast<size_t>(row) * k;
  float sum = 0.0f;
  // A lane's 16 bytes lie inside one 128-block (8 lanes per block, 4 blocks per 512-byte step).
  for (uint32_t column = lane * 16u; column < k; column += 512u) {
    const uint4 w = load_streaming_16(weight_row + column);
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(input + column));
    const uint32_t block = column / 128u;
    const float scale = __ldg(input_scales + block) *
                        __ldg(weight_scales + row / 128u + static_cast<size_t>(block) * blocks_n);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
    float partial = 0.0f;
#pragma unroll
    for (int word = 0; word < 4; ++word) {
      const float2 w_low = decode_pair(ws[word] & 0xffffu), w_high = decode_pair(ws[word] >> 16);
      const float2 x_low = decode_pair(xs[word] & 0xffffu), x_high = decode_pair(xs[word] >> 16);
      partial = fmaf(x_low.x, w_low.x, partial);
      partial = fmaf(x_low.y, w_low.y, partial);
      partial = fmaf(x_high.x, w_high.x, partial);
      partial = fmaf(x_high.y, w_high.y, partial);
    }
    sum = fmaf(partial, scale, sum);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
  if (lane == 0u) output[row] = __float2bfloat16_rn(sum);
}

}  // namespace fp8_vector
}  // namespace mircuda_b200

extern "C" int mircuda_fp8_vector_create(int n, int k, void* stream, void** output) {
  using namespace mircuda_b200::fp8_vector;
  if (n <= 0 || k <= 0 || n % 128 != 0 || k % 128 != 0 || stream == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{n, k, static_cast<cudaStream_t>(stream)};
  if (plan == nullptr) return -2;
  *output = plan;
  return 0;
}

extern "C" size_t mircuda_fp8_vector_workspace_bytes(const void*) { return 0; }

extern "C" int mircuda_fp8_vector_execute(void* raw, void* stream, const void* input,
                                          const void* input_scales, const void* weight,
                                          const void* weight_scales, void* output) {
  using namespace mircuda_b200::fp8_vector;
  if (raw == nullptr || stream == nullptr || input == nullptr || input_scales == nullptr ||
      weight == nullptr || weight_scales == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight)) & 15u) != 0u) {
    return -1;
  }
  fp8_vector_kernel<<<(plan->n + kWarps - 1) / kWarps, kWarps * 32, 0, cuda_stream>>>(
      static_cast<const uint8_t*>(input), static_cast<const float*>(input_scales),
      static_cast<const uint8_t*>(weight), static_cast<const float*>(weight_scales),
      static_cast<__nv_bfloat16*>(output), static_cast<uint32_t>(plan->n),
      static_cast<uint32_t>(plan->k));
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" void mircuda_fp8_vector_destroy(void* raw) {
  delete static_cast<mircuda_b200::fp8_vector::Plan*>(raw);
}
