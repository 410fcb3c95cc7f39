// FP8 (e4m3) matmul with per-token and per-tensor / per-output-channel scales and an optional
// bias: t = float(weight_scale[n or 0]) * sum_k x[m,k] * w[n,k];
// y[m,n] = bf16(has_bias ? fma(input_scale[m], t, float(bias[n])) : input_scale[m] * t),
// fp32 accumulation. Replaces the reference's CUTLASS plans (sys/native/scaled_fp8_sm120.cuh:21-71
// for the epilogue tree, sys/native/scaled_fp8_sm120.cu:125-206 for the entry points) behind
// the same C entry points. Input scales are fp32; weight scales are fp32 or bf16 (scale_type),
// one for the tensor or one per output channel (weight_scale_type); n and k are multiples of 16.
//
// Up to 16 tokens (the reference's decode tiles; its tile argument is accepted and has no
// meaning here) the op streams N*K weight bytes once and is bound by HBM: a 256-thread CTA owns
// 16 weight rows, its 8 warps interleave over 64-byte pieces of K, every lane loads 16 bytes of
// two weight rows with streaming loads and feeds them to mma.sync.m16n8k32 (e4m3, weights on
// the 16-row side, tokens on the 8-column side, a second instruction for tokens 8-15); the
// warps' partial sums meet in shared memory and thread (token, row) applies the epilogue.
// More tokens run the persistent tcgen05 tile kernel of dense_tile.cuh with kind::f8f6f4,
// 128 x 256 tiles and 128 elements of K per stage; this file supplies its epilogue.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <new>

#include <cstdlib>

#include "dense_pair.cuh"
#include "dense_tile.cuh"
#include "fp4_codec.cuh"
#include "ptx.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace scaled_fp8 {

using dense_tile::dense_tile_kernel;
using dense_tile::kBlockM;
using dense_tile::kThreads;
using dense_tile::Layout;

constexpr uint32_t kBlockN = 256, kStages = 4, kAccStages = 2;
constexpr uint32_t kPairStages = 6;     // a CTA of a pair holds 32 KB per stage
constexpr int kRowsWarps = 8;
constexpr int kRowsUnroll = 4;

struct Scales {
  const float* input_scales;
  const void* weight_scales;
  const __nv_bfloat16* bias;     // null without a bias
  bool bf16_scales;
  bool tensor_scale;

  __device__ __forceinline__ float weight_scale(uint32_t column) const {
    const uint32_t index = tensor_scale ? 0u : column;
    return bf16_scales ? __bfloat162float(static_cast<const __nv_bfloat16*>(weight_scales)[index])
                       : static_cast<const float*>(weight_scales)[index];
  }

  __device__ __forceinline__ float finish(float sum, float input_scale, uint32_t column) const {
    const float scaled = __fmul_rn(weight_scale(column), sum);
    return bias != nullptr ? fmaf(input_scale, scaled, __bfloat162float(bias[column]))
                           : __fmul_rn(input_scale, scaled);
  }
};

// Epilogue of the tile kernel: 32 consecutive accumulator columns of one row per call.
struct Epilogue {
  static constexpr uint32_t kElementBytes = 1u;
  __nv_bfloat16* output;
  Scales scales;

  __device__ __forceinline__ void store(uint32_t row, uint32_t column, const uint32_t (&values)[32],
                                        uint32_t n) const {
    const float input_scale = scales.input_scales[row];
    const size_t base = static_cast<size_t>(row) * n + column;
    // n is a multiple of 16: the 32 columns are all inside the row or exactly half of them are.
    const uint32_t parts = column + 32u <= n ? 4u : 2u;
#pragma unroll
    for (uint32_t part = 0; part < 4u; ++part) {
      if (part < parts) {
        uint32_t packed[4];
#pragma unroll
        for (uint32_t pair = 0; pair < 4u; ++pair) {
          const uint32_t item = part * 8u + pair * 2u;
          const float low = scales.finish(__uint_as_float(values[item]), input_scale, column + item);
          const float high =
              scales.finish(__uint_as_float(values[item + 1u]), input_scale, column + item + 1u);
          const __nv_bfloat162 two = __floats2bfloat162_rn(low, high);
          packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
        }
        reinterpret_cast<uint4*>(output + base)[part] =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
  }
};

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Up to 16 tokens. Grid: n / 16 CTAs of 8 warps. A 64-byte piece of K is split over the four
// lanes of a quad, 16 bytes each; which of those bytes meets which is the same for the weight
// and the token operand, so the instruction's own K order does not matter.
template <bool SECOND_HALF>
__global__ void __launch_bounds__(kRowsWarps * 32)
scaled_fp8_rows_kernel(const uint8_t* __restrict__ input, const uint8_t* __restrict__ weight,
                       __nv_bfloat16* __restrict__ output, const Scales scales, uint32_t m,
                       uint32_t n, uint32_t k) {
  __shared__ float partial[kRowsWarps][16][17];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t group = lane >> 2, quad = lane & 3u;
  const uint32_t n0 = blockIdx.x * 16u;
  const uint8_t* weight_low = weight + static_cast<size_t>(n0 + group) * k + quad * 16u;
  const uint8_t* weight_high = weight_low + static_cast<size_t>(8u) * k;
  const uint8_t* token_low = input + static_cast<size_t>(group) * k + quad * 16u;
  const uint8_t* token_high = token_low + static_cast<size_t>(8u) * k;
  const bool low_valid = group < m;
  const bool high_valid = SECOND_HALF && group + 8u < m;
  float first[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float second[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  for (uint32_t offset = warp * 64u; offset < k; offset += kRowsWarps * kRowsUnroll * 64u) {
    uint4 w_low[kRowsUnroll], w_high[kRowsUnroll], x_low[kRowsUnroll], x_high[kRowsUnroll];
#pragma unroll
    for (int step = 0; step < kRowsUnroll; ++step) {
      const uint32_t at = offset + step * kRowsWarps * 64u;
      const bool inside = at + quad * 16u < k;
      w_low[step] = inside ? load_streaming_16(weight_low + at) : zero;
      w_high[step] = inside ? load_streaming_16(weight_high + at) : zero;
      x_low[step] = inside && low_valid ? __ldg(reinterpret_cast<const uint4*>(token_low + at)) : zero;
      if (SECOND_HALF) {
        x_high[step] =
            inside && high_valid ? __ldg(reinterpret_cast<const uint4*>(token_high + at)) : zero;
      }
    }
#pragma unroll
    for (int step = 0; step < kRowsUnroll; ++step) {
      mma_e4m3(first, w_low[step].x, w_high[step].x, w_low[step].y, w_high[step].y, x_low[step].x,
               x_low[step].y);
      mma_e4m3(first, w_low[step].z, w_high[step].z, w_low[step].w, w_high[step].w, x_low[step].z,
               x_low[step].w);
      if (SECOND_HALF) {
        mma_e4m3(second, w_low[step].x, w_high[step].x, w_low[step].y, w_high[step].y,
                 x_high[step].x, x_high[step].y);
        mma_e4m3(second, w_low[step].z, w_high[step].z, w_low[step].w, w_high[step].w,
                 x_high[step].z, x_high[step].w);
      }
    }
  }

  // Accumulator element i of a lane: weight row group + 8 * (i / 2), token 2 * quad + i % 2.
#pragma unroll
  for (int item = 0; item < 4; ++item) {
    const uint32_t row = group + 8u * (item >> 1), token = 2u * quad + (item & 1);
    partial[warp][token][row] = first[item];
    partial[warp][token + 8u][row] = SECOND_HALF ? second[item] : 0.0f;
  }
  __syncthreads();
  const uint32_t token = threadIdx.x >> 4, row = threadIdx.x & 15u;
  if (token < m) {
    float sum = 0.0f;
#pragma unroll
    for (int from = 0; from < kRowsWarps; ++from) sum += partial[from][token][row];
    output[static_cast<size_t>(token) * n + n0 + row] =
        __float2bfloat16_rn(scales.finish(sum, scales.input_scales[token], n0 + row));
  }
}

struct Plan {
  int m, n, k;
  bool bf16_scales, tensor_scale, has_bias;
  int sm_count;
  cudaStream_t stream;
  uint32_t* status;          // pinned; set by the tile kernel when a wait gives up
  const void* cached_input;
  const void* cached_weight;
  CUtensorMap map_input, map_weight;
  bool pair;                // more than 128 tokens: CTA pairs (dense_pair.cuh)
  int resident_pairs;
};

}  // namespace scaled_fp8
}  // namespace mircuda_b200

extern "C" int mircuda_scaled_fp8_create(int m, int n, int k, int scale_type, int weight_scale_type,
                                         int has_bias, int tile, void* stream, void** output) {
  using namespace mircuda_b200::scaled_fp8;
  if (m <= 0 || n <= 0 || k <= 0 || n % 16 != 0 || k % 16 != 0 ||
      (scale_type != 0 && scale_type != 1) || (weight_scale_type != 0 && weight_scale_type != 1) ||
      (tile != 0 && tile != 1) || stream == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->m = m;
  plan->n = n;
  plan->k = k;
  plan->bf16_scales = scale_type == 1;
  plan->tensor_scale = weight_scale_type == 0;
  plan->has_bias = has_bias != 0;
  plan->stream = static_cast<cudaStream_t>(stream);
  int device = 0;
  int status = static_cast<int>(cudaGetDevice(&device));
  if (status == 0) {
    status = static_cast<int>(
        cudaDeviceGetAttribute(&plan->sm_count, cudaDevAttrMultiProcessorCount, device));
  }
  if (status == 0) {
    status = static_cast<int>(cudaHostAlloc(reinterpret_cast<void**>(&plan->status),
                                            sizeof(uint32_t), cudaHostAllocMapped));
  }
  if (status == 0) {
    status = static_cast<int>(cudaFuncSetAttribute(
        dense_tile_kernel<kBlockN, kStages, kAccStages, Epilogue>,
        cudaFuncAttributeMaxDynamicSharedMemorySize,
        Layout<kBlockN, kStages, kAccStages>::kDynamicBytes));
  }
  // More than 128 tokens run on CTA pairs (MIRCUDA_B200_DENSE_PAIR=0 keeps single CTAs).
  const char* pair_choice = std::getenv("MIRCUDA_B200_DENSE_PAIR");
  plan->pair = m > static_cast<int>(kBlockM) && !(pair_choice != nullptr && pair_choice[0] == '0');
  if (status == 0 && plan->pair) {
    status = mircuda_b200::dense_pair::prepare<kBlockN, kPairStages, kAccStages, Epilogue>(plan->sm_count, &plan->resident_pairs);
  }
  if (status != 0) {
    if (plan->status != nullptr) cudaFreeHost(plan->status);
    delete plan;
    return status;
  }
  *plan->status = 0u;
  *output = plan;
  return 0;
}

extern "C" size_t mircuda_scaled_fp8_workspace_bytes(const void*) { return 0; }

extern "C" int mircuda_scaled_fp8_execute(void* raw, void* stream, const void* input,
                                          const void* weight, const float* input_scales,
                                          const void* weight_scales, const void* bias,
                                          void* output) {
  using namespace mircuda_b200;
  using namespace mircuda_b200::scaled_fp8;
  if (raw == nullptr || stream == nullptr || input == nullptr || weight == nullptr ||
      input_scales == nullptr || weight_scales == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  if ((bias != nullptr) != plan->has_bias) return -1;
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight) |
        reinterpret_cast<uintptr_t>(output)) & 15u) != 0u) {
    return -1;
  }
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  const Scales scales{input_scales, weight_scales, static_cast<const __nv_bfloat16*>(bias),
                      plan->bf16_scales, plan->tensor_scale};
  auto* result = static_cast<__nv_bfloat16*>(output);
  if (plan->m <= 16) {
    const unsigned int grid = static_cast<unsigned int>(plan->n / 16);
    if (plan->m > 8) {
      scaled_fp8_rows_kernel<true><<<grid, kRowsWarps * 32, 0, cuda_stream>>>(
          static_cast<const uint8_t*>(input), static_cast<const uint8_t*>(weight), result, scales,
          plan->m, plan->n, plan->k);
    } else {
      scaled_fp8_rows_kernel<false><<<grid, kRowsWarps * 32, 0, cuda_stream>>>(
          static_cast<const uint8_t*>(input), static_cast<const uint8_t*>(weight), result, scales,
          plan->m, plan->n, plan->k);
    }
    return static_cast<int>(cudaPeekAtLastError());
  }
  if (input != plan->cached_input) {
    const int status = encode_k_major_map(&plan->map_input, input, plan->m, plan->k, 1u, kBlockM);
    if (status != 0) return status;
    plan->cached_input = input;
  }
  if (weight != plan->cached_weight) {
    const int status = encode_k_major_map(&plan->map_weight, weight, plan->n, plan->k, 1u,
                                          plan->pair ? kBlockN / 2u : kBlockN);
    if (status != 0) return status;
    plan->cached_weight = weight;
  }
  if (plan->pair) {
    return mircuda_b200::dense_pair::launch<kBlockN, kPairStages, kAccStages, Epilogue>(
        cuda_stream, plan->resident_pairs, plan->map_input, plan->map_weight, plan->m, plan->n, plan->k,
        ptx::make_f16_idesc(false, 2u * kBlockM, kBlockN), Epilogue{result, scales}, plan->status);
  }
  const uint32_t tiles = ((plan->m + kBlockM - 1u) / kBlockM) * ((plan->n + kBlockN - 1u) / kBlockN);
  const uint32_t grid = tiles < static_cast<uint32_t>(plan->sm_count) ? tiles : plan->sm_count;
  const uint32_t idesc = ptx::make_f16_idesc(false, kBlockM, kBlockN);
  dense_tile_kernel<kBlockN, kStages, kAccStages, Epilogue>
      <<<grid, kThreads, Layout<kBlockN, kStages, kAccStages>::kDynamicBytes, cuda_stream>>>(
          plan->map_input, plan->map_weight, plan->m, plan->n, plan->k, idesc,
          Epilogue{result, scales}, plan->status);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" void mircuda_scaled_fp8_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::scaled_fp8::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
