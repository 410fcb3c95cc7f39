// Weight-only MXFP8 projection: out[t, n] = bf16(sum_k x[t, k] * e4m3(w[n, k]) * 2^(s[n, k/32] - 127))
// with bf16 activations that are NOT quantised, E4M3 weights handed over as little-endian
// u32 words and row-major [N, K/32] E8M0 scales. Replaces the reference's run-time-compiled
// kernels `mircuda_mxfp8_bf16` / `mircuda_mxfp8_bf16_tiled` (kernels/mxfp8.cu:111-217) and
// their launches (src/mxfp8/matmul.rs:131-157).
//
// For decode-sized token counts the op is bound by streaming the weights (N*K bytes). One
// warp owns one output row and up to four tokens; each lane reads 16 weight bytes per step
// with a streaming 16-byte load (the reference reads single bytes) and keeps eight such loads
// in flight, decodes them with the hardware e4m3x2 -> f16x2 conversion (exact) and accumulates
// in fp32, applying the block scale once per 16 products. The order of the sums is the same
// whatever the look-ahead. Up to eight tokens with K a multiple of 128 and N a multiple of 16
// take the tensor-core kernel further down instead, which spends a third of the conversions.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>

#include "fp4_codec.cuh"

namespace mircuda_b200 {
namespace {

constexpr int kWarps = 8;
constexpr int kTokenTile = 4;
constexpr int kAhead = 8;        // steps of a lane's row whose loads are in flight together

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
    const uint8_t* scale_row = scales + static_cast<size_t>(row) * groups;
    // A lane's loads of kAhead steps (16 weight bytes and one scale byte each, 512 columns apart)
    // are all issued before the first of them is used: with one load in flight per lane the
    // kernel waited for memory latency, not for bandwidth.
    for (uint32_t base = lane * 16u; base < k; base += kAhead * 512u) {
      uint4 ahead[kAhead];
      uint32_t exponents[kAhead];
#pragma unroll
      for (int step = 0; step < kAhead; ++step) {
        const uint32_t column = base + step * 512u;
        if (column < k) {
          ahead[step] = load_streaming_16(weight_row + column);
          exponents[step] = scale_row[column / 32u];
        }
      }
#pragma unroll
      for (int step = 0; step < kAhead; ++step) {
        const uint32_t column = base + step * 512u;
        if (column >= k) break;
        const uint4 packed = ahead[step];
        const uint32_t exponent = exponents[step];
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


// Up to eight tokens on the tensor cores: a CTA owns 16 output rows, its eight warps take the
// 128-column pieces of K in turn. Per 32-column scale block a lane loads 8 weight bytes of rows
// g and g + 8 (g = lane / 4) at byte 8 * (lane % 4), so a warp instruction reads whole 32-byte
// sectors; the block is two m16n8k16 steps (step j uses the lane's bytes 4 j .. 4 j + 3) whose
// K order is the same permutation on the weight and the activation side, so no data is moved
// between lanes. Weights go e4m3x2 -> f16x2 (exact), activations bf16 -> f16 (exact between
// 2^-14 and 65504, saturating above), products accumulate in fp32 inside the MMA and the block's
// power-of-two scale multiplies the sum of the two steps in fp32.
constexpr int kMmaWarps = 8;
constexpr int kMmaRows = 16;

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_codes) {
  uint32_t pair;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(static_cast<uint16_t>(two_codes)));
  return pair;
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t pair) {
  uint32_t d;
  const float low = __uint_as_float(pair << 16);
  const float high = __uint_as_float(pair & 0xffff0000u);
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(high), "f"(low));
  return d;
}

__device__ __forceinline__ void mma_f16_16x8x16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                                const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ uint2 load_streaming_8(const void* pointer) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(pointer));
  return v;
}

__device__ __forceinline__ float e8m0_scale(uint32_t exponent) {
  return exponent == 0u ? 5.87747175e-39f : __uint_as_float(exponent << 23);
}

__global__ void __launch_bounds__(kMmaWarps * 32)
mxfp8_weight_only_mma_kernel(const __nv_bfloat16* __restrict__ input, const uint8_t* __restrict__ weight,
                             const uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ output,
                             uint32_t tokens, uint32_t k, uint32_t n) {
  __shared__ float partial[kMmaWarps][kMmaRows][8];
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, q = lane & 3u;
  const uint32_t row0 = blockIdx.x * kMmaRows;
  const uint32_t groups = k / 32u;
  const uint8_t* upper = weight + static_cast<size_t>(row0 + g) * k + q * 8u;
  const uint8_t* lower = upper + static_cast<size_t>(8u) * k;
  const uint8_t* upper_scales = scales + static_cast<size_t>(row0 + g) * groups;
  const uint8_t* lower_scales = upper_scales + static_cast<size_t>(8u) * groups;
  const bool has_token = g < tokens;
  const __nv_bfloat16* x = input + static_cast<size_t>(has_token ? g : 0u) * k + q * 8u;

  float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // Two pieces per round: the loads of both (128 weight bytes per lane) are issued before the
  // first is used.
  constexpr int kPieces = 2;
  for (uint32_t first_piece = warp; first_piece * 4u < groups; first_piece += kPieces * kMmaWarps) {
    uint2 high[kPieces][4], low[kPieces][4];
    uint32_t upper_word[kPieces], lower_word[kPieces];
#pragma unroll
    for (int slot = 0; slot < kPieces; ++slot) {
      const uint32_t piece = first_piece + slot * kMmaWarps;
      if (piece * 4u >= groups) break;
      const uint32_t column = piece * 128u;
#pragma unroll
      for (int block = 0; block < 4; ++block) {
        high[slot][block] = load_streaming_8(upper + column + block * 32);
        low[slot][block] = load_streaming_8(lower + column + block * 32);
      }
      upper_word[slot] = *reinterpret_cast<const uint32_t*>(upper_scales + piece * 4u);
      lower_word[slot] = *reinterpret_cast<const uint32_t*>(lower_scales + piece * 4u);
    }
#pragma unroll
    for (int slot = 0; slot < kPieces; ++slot) {
      const uint32_t piece = first_piece + slot * kMmaWarps;
      if (piece * 4u >= groups) break;
#pragma unroll
      for (int block = 0; block < 4; ++block) {
        const uint2 h = high[slot][block], l = low[slot][block];
        // the activations are a few KB per token and stay in L1
        const uint4 v = has_token ? __ldg(reinterpret_cast<const uint4*>(x + piece * 128u + block * 32))
                                  : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t first[4] = {e4m3x2_to_f16x2(h.x & 0xffffu), e4m3x2_to_f16x2(l.x & 0xffffu),
                                   e4m3x2_to_f16x2(h.x >> 16), e4m3x2_to_f16x2(l.x >> 16)};
        const uint32_t second[4] = {e4m3x2_to_f16x2(h.y & 0xffffu), e4m3x2_to_f16x2(l.y & 0xffffu),
                                    e4m3x2_to_f16x2(h.y >> 16), e4m3x2_to_f16x2(l.y >> 16)};
        float d[4];
        mma_f16_16x8x16(d, first, bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), zero);
        mma_f16_16x8x16(d, second, bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w), d);
        const float upper_scale = e8m0_scale((upper_word[slot] >> (8 * block)) & 0xffu);
        const float lower_scale = e8m0_scale((lower_word[slot] >> (8 * block)) & 0xffu);
        sums[0] = fmaf(upper_scale, d[0], sums[0]);
        sums[1] = fmaf(upper_scale, d[1], sums[1]);
        sums[2] = fmaf(lower_scale, d[2], sums[2]);
        sums[3] = fmaf(lower_scale, d[3], sums[3]);
      }
    }
  }
  partial[warp][g][q * 2u] = sums[0];
  partial[warp][g][q * 2u + 1u] = sums[1];
  partial[warp][g + 8u][q * 2u] = sums[2];
  partial[warp][g + 8u][q * 2u + 1u] = sums[3];
  __syncthreads();
  if (threadIdx.x < kMmaRows * 8u) {
    const uint32_t row = threadIdx.x & 15u, token = threadIdx.x >> 4;
    float total = 0.0f;
#pragma unroll
    for (int other = 0; other < kMmaWarps; ++other) total += partial[other][row][token];
    if (token < tokens) output[static_cast<size_t>(token) * n + row0 + row] = __float2bfloat16_rn(total);
  }
}


// The same kernel for one or two tokens: the CTA first converts the tokens' activations to f16 into
// shared memory (tokens * k * 2 bytes of dynamic shared memory) while its first weight loads are in
// flight; a lane then reads the eight f16 values of a block with one 16-byte shared load instead of
// converting them itself (a quarter of the instructions of a block).
__global__ void __launch_bounds__(kMmaWarps * 32)
mxfp8_weight_only_staged_kernel(const __nv_bfloat16* __restrict__ input, const uint8_t* __restrict__ weight,
                             const uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ output,
                             uint32_t tokens, uint32_t k, uint32_t n) {
  __shared__ float partial[kMmaWarps][kMmaRows][8];
  extern __shared__ __align__(16) uint4 staged[];          // [token][k / 8] of eight f16 each
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, q = lane & 3u;
  const uint32_t row0 = blockIdx.x * kMmaRows;
  const uint32_t groups = k / 32u;
  const uint8_t* upper = weight + static_cast<size_t>(row0 + g) * k + q * 8u;
  const uint8_t* lower = upper + static_cast<size_t>(8u) * k;
  const uint8_t* upper_scales = scales + static_cast<size_t>(row0 + g) * groups;
  const uint8_t* lower_scales = upper_scales + static_cast<size_t>(8u) * groups;
  const bool has_token = g < tokens;
  const uint4* staged_x = staged + static_cast<size_t>(has_token ? g : 0u) * (k / 8u) + q;

  float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // Two pieces per round: the loads of both (128 weight bytes per lane) are issued before the
  // first is used.
  constexpr int kPieces = 2;
  uint2 high[kPieces][4], low[kPieces][4];
  uint32_t upper_word[kPieces], lower_word[kPieces];
  auto load_round = [&](uint32_t first_piece) {
#pragma unroll
    for (int slot = 0; slot < kPieces; ++slot) {
      const uint32_t piece = first_piece + slot * kMmaWarps;
      if (piece * 4u >= groups) break;
      const uint32_t column = piece * 128u;
#pragma unroll
      for (int block = 0; block < 4; ++block) {
        high[slot][block] = load_streaming_8(upper + column + block * 32);
        low[slot][block] = load_streaming_8(lower + column + block * 32);
      }
      upper_word[slot] = *reinterpret_cast<const uint32_t*>(upper_scales + piece * 4u);
      lower_word[slot] = *reinterpret_cast<const uint32_t*>(lower_scales + piece * 4u);
    }
  };
  auto use_round = [&](uint32_t first_piece) {
#pragma unroll
    for (int slot = 0; slot < kPieces; ++slot) {
      const uint32_t piece = first_piece + slot * kMmaWarps;
      if (piece * 4u >= groups) break;
#pragma unroll
      for (int block = 0; block < 4; ++block) {
        const uint2 h = high[slot][block], l = low[slot][block];
        const uint4 v = has_token ? staged_x[piece * 16u + block * 4] : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t b[4] = {v.x, v.y, v.z, v.w};
        const uint32_t first[4] = {e4m3x2_to_f16x2(h.x & 0xffffu), e4m3x2_to_f16x2(l.x & 0xffffu),
                                   e4m3x2_to_f16x2(h.x >> 16), e4m3x2_to_f16x2(l.x >> 16)};
        const uint32_t second[4] = {e4m3x2_to_f16x2(h.y & 0xffffu), e4m3x2_to_f16x2(l.y & 0xffffu),
                                    e4m3x2_to_f16x2(h.y >> 16), e4m3x2_to_f16x2(l.y >> 16)};
        float d[4];
        mma_f16_16x8x16(d, first, b[0], b[1], zero);
        mma_f16_16x8x16(d, second, b[2], b[3], d);
        const float upper_scale = e8m0_scale((upper_word[slot] >> (8 * block)) & 0xffu);
        const float lower_scale = e8m0_scale((lower_word[slot] >> (8 * block)) & 0xffu);
        sums[0] = fmaf(upper_scale, d[0], sums[0]);
        sums[1] = fmaf(upper_scale, d[1], sums[1]);
        sums[2] = fmaf(lower_scale, d[2], sums[2]);
        sums[3] = fmaf(lower_scale, d[3], sums[3]);
      }
    }
  };
  {
    load_round(warp);
    const uint32_t vectors = tokens * (k / 8u);
    const uint4* source = reinterpret_cast<const uint4*>(input);
    for (uint32_t index = threadIdx.x; index < vectors; index += kMmaWarps * 32u) {
      const uint4 v = __ldg(source + index);
      staged[index] = make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z),
                                 bf16x2_to_f16x2(v.w));
    }
    __syncthreads();
  }
  for (uint32_t first_piece = warp; first_piece * 4u < groups; first_piece += kPieces * kMmaWarps) {
    use_round(first_piece);
    load_round(first_piece + kPieces * kMmaWarps);
  }
  partial[warp][g][q * 2u] = sums[0];
  partial[warp][g][q * 2u + 1u] = sums[1];
  partial[warp][g + 8u][q * 2u] = sums[2];
  partial[warp][g + 8u][q * 2u + 1u] = sums[3];
  __syncthreads();
  if (threadIdx.x < kMmaRows * 8u) {
    const uint32_t row = threadIdx.x & 15u, token = threadIdx.x >> 4;
    float total = 0.0f;
#pragma unroll
    for (int other = 0; other < kMmaWarps; ++other) total += partial[other][row][token];
    if (token < tokens) output[static_cast<size_t>(token) * n + row0 + row] = __float2bfloat16_rn(total);
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
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  const uintptr_t addresses = reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight);
  // MIRCUDA_B200_MXFP8_WEIGHT_ONLY=simt keeps every shape on the fp32 kernel (activations beyond
  // the f16 range, which the tensor-core kernel saturates at 65504).
  static const bool simt_only = [] {
    const char* value = std::getenv("MIRCUDA_B200_MXFP8_WEIGHT_ONLY");
    return value != nullptr && value[0] == 's';
  }();
  if (!simt_only && tokens <= 8u && input_features % 128u == 0u && output_features % kMmaRows == 0u &&
      (addresses & 15u) == 0u && (reinterpret_cast<uintptr_t>(scales) & 3u) == 0u) {
    // Activations staged in shared memory as f16 for one or two tokens of up to 32 KB (measured at
    // K = 4096 and 12288: M = 1 gains 5-17 %, M = 4 loses as much to the staging itself); converted
    // in registers otherwise.
    const size_t staged_bytes = static_cast<size_t>(tokens) * input_features * 2u;
    if (tokens <= 2u && staged_bytes <= 32768u) {
      mxfp8_weight_only_staged_kernel<<<output_features / kMmaRows, kMmaWarps * 32, staged_bytes, cuda_stream>>>(
          static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
          static_cast<const uint8_t*>(scales), static_cast<__nv_bfloat16*>(output), tokens, input_features,
          output_features);
    } else {
      mxfp8_weight_only_mma_kernel<<<output_features / kMmaRows, kMmaWarps * 32, 0, cuda_stream>>>(
          static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
          static_cast<const uint8_t*>(scales), static_cast<__nv_bfloat16*>(output), tokens, input_features,
          output_features);
    }
    return static_cast<int>(cudaPeekAtLastError());
  }
  const dim3 grid((output_features + kWarps - 1) / kWarps, (tokens + kTokenTile - 1) / kTokenTile);
  if (grid.y > 65535u) return -1;
  mxfp8_weight_only_kernel<<<grid, kWarps * 32, 0, cuda_stream>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
      static_cast<const uint8_t*>(scales), static_cast<__nv_bfloat16*>(output), tokens,
      input_features, output_features);
  return static_cast<int>(cudaPeekAtLastError());
}
