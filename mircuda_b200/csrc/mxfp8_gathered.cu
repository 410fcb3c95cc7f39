// Routed weight-only MXFP8 projection and MXFP8 embedding lookup (decode path of MXFP8
// checkpoints). Replace the reference's run-time-compiled kernels
// `mircuda_mxfp8_bf16_gathered` (kernels/mxfp8.cu:219-271, launched from src/mxfp8/gathered.rs)
// and `mircuda_mxfp8_embedding_bf16` (kernels/mxfp8.cu:273-296) with ahead-of-time launchers.
//
// gathered: for every assignment a (input row a / selections_per_input, matrix selected[a]):
//   out[a, r] = bf16(sum_c x[c] * e4m3(W[matrix, r, c]) * 2^(s[matrix, r, c/32] - 127) (+ bias[matrix, r]))
//   and 0 where the matrix index is out of range. Bound by streaming the selected weight rows:
//   one warp per (assignment, output row), 16 weight bytes per lane and step with a streaming
//   16-byte load (the reference reads single bytes), hardware e4m3x2 -> f16x2 decoding (exact),
//   fp32 accumulation with the block scale applied once per 16 products.
// embedding: out[t, c] = bf16(e4m3(W[row, c]) * 2^(s[row, c/32] - 127) * output_scale) for
//   row = selected[selected_start + t]; rows >= vocab are left untouched. Same expression and
//   rounding order as the reference, so results are bit-identical; 16 columns per thread.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "fp4_codec.cuh"

namespace mircuda_b200 {
namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ float2 decode_pair(uint32_t two_codes) {
  uint32_t pair;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(static_cast<uint16_t>(two_codes)));
  return __half22float2(*reinterpret_cast<const __half2*>(&pair));
}

__device__ __forceinline__ float e8m0(uint32_t exponent) {   // 2^(e-127); e = 0 is subnormal
  return exponent == 0u ? 5.87747175e-39f : __uint_as_float(exponent << 23);
}

__device__ __forceinline__ void decode16(const uint4& packed, float (&w)[16]) {
  const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
  for (int word = 0; word < 4; ++word) {
    const float2 low = decode_pair(words[word] & 0xffffu);
    const float2 high = decode_pair(words[word] >> 16);
    w[word * 4 + 0] = low.x;
    w[word * 4 + 1] = low.y;
    w[word * 4 + 2] = high.x;
    w[word * 4 + 3] = high.y;
  }
}

__global__ void __launch_bounds__(kWarps * 32)
mxfp8_gathered_kernel(const __nv_bfloat16* __restrict__ input, const uint8_t* __restrict__ weight,
                      const uint8_t* __restrict__ scales, const __nv_bfloat16* __restrict__ bias,
                      const uint32_t* __restrict__ selected, __nv_bfloat16* __restrict__ output,
                      uint32_t assignments, uint32_t matrices, uint32_t rows, uint32_t columns,
                      uint32_t selections_per_input, bool has_bias) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  const uint32_t assignment = blockIdx.y;
  if (row >= rows || assignment >= assignments) return;
  const uint32_t matrix = __ldg(selected + assignment);
  if (matrix >= matrices) {
    if (lane == 0u) output[static_cast<size_t>(assignment) * rows + row] = __float2bfloat16_rn(0.0f);
    return;
  }
  const size_t matrix_row = static_cast<size_t>(matrix) * rows + row;
  const uint32_t groups = columns / 32u;
  const __nv_bfloat16* x_row = input + static_cast<size_t>(assignment / selections_per_input) * columns;
  const uint8_t* weight_row = weight + matrix_row * columns;
  float sum = 0.0f;
  if ((columns & 15u) == 0u && (reinterpret_cast<uintptr_t>(weight) & 15u) == 0u &&
      (reinterpret_cast<uintptr_t>(input) & 15u) == 0u) {
    for (uint32_t column = lane * 16u; column < columns; column += 512u) {
      const uint4 packed = load_streaming_16(weight_row + column);
      const float block_scale = e8m0(scales[matrix_row * groups + column / 32u]);
      float w[16];
      decode16(packed, w);
      const uint4* x = reinterpret_cast<const uint4*>(x_row + column);
      const uint4 first = __ldg(x);
      const uint4 second = __ldg(x + 1);
      const uint32_t xs[8] = {first.x, first.y, first.z, first.w, second.x, second.y, second.z, second.w};
      float partial = 0.0f;
#pragma unroll
      for (int pair = 0; pair < 8; ++pair) {
        partial = fmaf(__uint_as_float(xs[pair] << 16), w[pair * 2], partial);
        partial = fmaf(__uint_as_float(xs[pair] & 0xffff0000u), w[pair * 2 + 1], partial);
      }
      sum = fmaf(partial, block_scale, sum);
    }
  } else {
    for (uint32_t column = lane; column < columns; column += 32u) {
      const float w = decode_pair(weight_row[column]).x * e8m0(scales[matrix_row * groups + column / 32u]);
      sum = fmaf(__bfloat162float(x_row[column]), w, sum);
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
  if (lane == 0u) {
    if (has_bias) sum += __bfloat162float(bias[matrix_row]);
    output[static_cast<size_t>(assignment) * rows + row] = __float2bfloat16_rn(sum);
  }
}

// One thread per 16 columns (hidden % 16 == 0) or per column otherwise.
__global__ void __launch_bounds__(256)
mxfp8_embedding_kernel(const uint8_t* __restrict__ weight, const uint8_t* __restrict__ scales,
                       const uint32_t* __restrict__ selected, __nv_bfloat16* __restrict__ output,
                       uint32_t selected_start, uint32_t tokens, uint32_t vocab, uint32_t hidden,
                       float output_scale, bool vectors) {
  const uint32_t token = blockIdx.y;
  if (token >= tokens) return;
  const uint32_t row = __ldg(selected + selected_start + token);
  if (row >= vocab) return;
  const uint32_t groups = hidden / 32u;
  const uint8_t* weight_row = weight + static_cast<size_t>(row) * hidden;
  __nv_bfloat16* out_row = output + static_cast<size_t>(token) * hidden;
  const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
  if (vectors) {
    const uint32_t column = item * 16u;
    if (column >= hidden) return;
    const uint4 packed = load_streaming_16(weight_row + column);
    const float scale = e8m0(scales[static_cast<size_t>(row) * groups + column / 32u]);
    float w[16];
    decode16(packed, w);
    uint32_t words[8];
#pragma unroll
    for (int pair = 0; pair < 8; ++pair) {
      // (e4m3 * scale) * output_scale, in this order, each product rounded to fp32.
      const __nv_bfloat162 two = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(w[pair * 2], scale), output_scale),
                                                       __fmul_rn(__fmul_rn(w[pair * 2 + 1], scale), output_scale));
      words[pair] = *reinterpret_cast<const uint32_t*>(&two);
    }
    uint4* destination = reinterpret_cast<uint4*>(out_row + column);
    destination[0] = make_uint4(words[0], words[1], words[2], words[3]);
    destination[1] = make_uint4(words[4], words[5], words[6], words[7]);
  } else {
    if (item >= hidden) return;
    const float scale = e8m0(scales[static_cast<size_t>(row) * groups + item / 32u]);
    out_row[item] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(decode_pair(weight_row[item]).x, scale), output_scale));
  }
}

}  // namespace
}  // namespace mircuda_b200

extern "C" int mircuda_b200_mxfp8_bf16_gathered(const void* input, const void* weight,
                                                const void* scales, const void* bias,
                                                const void* selected, void* output,
                                                uint32_t assignments, uint32_t matrices,
                                                uint32_t rows, uint32_t columns,
                                                uint32_t selections_per_input, void* stream) {
  using namespace mircuda_b200;
  if (input == nullptr || weight == nullptr || scales == nullptr || selected == nullptr ||
      output == nullptr || stream == nullptr || assignments == 0u || matrices == 0u || rows == 0u ||
      columns == 0u || columns % 32u != 0u || selections_per_input == 0u || assignments > 65535u) {
    return -1;
  }
  const dim3 grid((rows + kWarps - 1) / kWarps, assignments);
  mxfp8_gathered_kernel<<<grid, kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
      static_cast<const uint8_t*>(scales), static_cast<const __nv_bfloat16*>(bias),
      static_cast<const uint32_t*>(selected), static_cast<__nv_bfloat16*>(output), assignments,
      matrices, rows, columns, selections_per_input, bias != nullptr);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" int mircuda_b200_mxfp8_embedding_bf16(const void* weight, const void* scales,
                                                 const void* selected, void* output,
                                                 uint32_t selected_start, uint32_t tokens,
                                                 uint32_t vocab, uint32_t hidden,
                                                 float output_scale, void* stream) {
  using namespace mircuda_b200;
  if (weight == nullptr || scales == nullptr || selected == nullptr || output == nullptr ||
      stream == nullptr || tokens == 0u || vocab == 0u || hidden == 0u || hidden % 32u != 0u ||
      tokens > 65535u) {
    return -1;
  }
  const bool vectors = (reinterpret_cast<uintptr_t>(weight) & 15u) == 0u &&
                       (reinterpret_cast<uintptr_t>(output) & 15u) == 0u;
  const uint32_t items = vectors ? hidden / 16u : hidden;
  const dim3 grid((items + 255u) / 256u, tokens);
  mxfp8_embedding_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(weight), static_cast<const uint8_t*>(scales),
      static_cast<const uint32_t*>(selected), static_cast<__nv_bfloat16*>(output), selected_start,
      tokens, vocab, hidden, output_scale, vectors);
  return static_cast<int>(cudaPeekAtLastError());
}
