// bf16-activation x NVFP4-weight skinny GEMM for decode, M <= 8:
//   y[m, n] = bf16(global * sum_k x[m, k] * e2m1(W[n, k]) * ue4m3(s[n, k / 16]))
// Weights [N, K/2] (two codes per byte, even k low) and swizzled UE4M3 scales use the same
// layouts as the FP4 x FP4 GEMV. This entry point has no counterpart in the reference's C
// ABI; the reference serves this shape through its Marlin NVFP4 dense path, whose numerics
// (exact weight * scale products, fp32 accumulation, global scale before the bf16 round)
// it follows.
//
// The op streams 0.5625*N*K bytes once and is bound by HBM, for every M up to 8: weights are
// the 16-row operand of mma.sync.m16n8k16 (bf16 in, fp32 out) and the tokens ride its
// 8-wide dimension, so decoding cost does not grow with M. A CTA owns 128 rows (one scale
// row tile) x 512 K-elements; warp w owns K sub-range (w % 4) * 128 for rows (w / 4) * 64 and
// keeps the activations of that sub-range in registers as ready-made B fragments. E2M1
// codes become bf16 by bit placement (value * 2^-126, the zero-exponent codes as bf16
// subnormals) and are multiplied by ue4m3(s) * 2^118 with one packed bf16 multiply, which
// is exact; the epilogue undoes the 2^-8. Because a dot product does not care about the
// order of its terms, the K order inside a 32-element chunk is whatever makes the bit
// placement cheapest, and the activations are staged in shared memory in that same order.
// K-slices meet through per-slice partial sums; the last slice to arrive for a row tile
// (a counter, no spinning) adds them in a fixed order and writes bf16.
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <new>

#include "fp4_codec.cuh"
#include "layout.cuh"

namespace mircuda_b200 {
namespace nvfp4_vector {

constexpr int kThreads = 256;
constexpr int kTileRows = 128;
constexpr int kTileK = 512;
constexpr int kAtomsPerTile = kTileK / 64;
constexpr int kAtomStride = 512 + 8;
constexpr int kMaxTokens = 8;
constexpr int kChunks = kTileK / 32;                 // 32-element chunks per K-slice
constexpr int kTokenStride = kTileK + 8;             // bf16 elements, padded

struct Plan {
  int m;
  int n;
  int k;
  int slices;
  cudaStream_t stream;
  float* partials;          // [slices][row_tiles * 128][8]
  unsigned int* counters;   // [row_tiles]
};

// Position of element j (0..31) of a chunk in the staged order: word w = j / 8 holds nibbles
// n0..n7; the decoder emits pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7).
__device__ __forceinline__ int staged_position(int j) {
  const int word = j >> 3;
  const int nibble = j & 7;
  return word * 8 + (nibble & 3) * 2 + (nibble >> 2);
}

// Eight E2M1 codes -> four bf16x2 holding value * 2^-126: sign to bit 15, the three
// exponent/mantissa bits to bf16 bits 8..6. out[p] = (nibble p, nibble p + 4).
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

// ue4m3(code) * 2^118 as a bf16 replicated in both halves (exact: 4 significant bits).
__device__ __forceinline__ uint32_t scale_multiplier(uint8_t code) {
  const float scaled = decode_ue4m3(code) * 3.32306998946228968e35f;  // 2^118
  const uint32_t high = __float_as_uint(scaled) >> 16;
  return high | (high << 16);
}

__global__ void __launch_bounds__(kThreads)
nvfp4_vector_kernel(const __nv_bfloat16* __restrict__ input, const uint8_t* __restrict__ weight,
       const uint8_t* __restrict__ weight_scales, __nv_bfloat16* __restrict__ output,
       float* __restrict__ partials, unsigned int* __restrict__ counters, int m, int n, int k,
       int slices, float global_scale) {
  __shared__ __align__(16) uint8_t shared_scales[kAtomsPerTile * kAtomStride];
  __shared__ __align__(16) __nv_bfloat16 shared_x[kMaxTokens * kTokenStride];
  __shared__ __align__(16) float shared_sums[4][kTileRows][kMaxTokens];
  __shared__ bool last_arrival;

  const int row_tile = blockIdx.x;
  const int slice = blockIdx.y;
  const int k_begin = slice * kTileK;
  const int atoms_k = k / 64;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int group = lane >> 2;                     // row inside a 16-row step / token index
  const int quad = lane & 3;                       // 32-element chunk inside the warp's range
  const int warp_k = warp & 3;
  const int warp_rows = warp >> 2;
  const int chunk = warp_k * 4 + quad;             // chunk of this thread inside the slice
  const int element = k_begin + chunk * 32;
  const bool active = element < k;

  // All weight loads of this thread first: 4 row steps x 2 rows x 16 bytes.
  uint4 packed[4][2];
#pragma unroll
  for (int step = 0; step < 4; ++step) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = row_tile * kTileRows + warp_rows * 64 + step * 16 + half * 8 + group;
      packed[step][half] = make_uint4(0u, 0u, 0u, 0u);
      if (active && row < n) {
        packed[step][half] =
            load_streaming_16(weight + (static_cast<size_t>(row) * k + element) / 2);
      }
    }
  }

  // Scale atoms of the tile (whole, coalesced) and the activation slice in staged order.
  {
    const int atom = threadIdx.x >> 5;
    const int offset = (threadIdx.x & 31) * 16;
    const int atom_column = k_begin / 64 + atom;
    uint4 value = make_uint4(0u, 0u, 0u, 0u);
    if (atom_column < atoms_k) {
      value = __ldg(reinterpret_cast<const uint4*>(
          weight_scales + (static_cast<size_t>(row_tile) * atoms_k + atom_column) * 512 + offset));
    }
    *reinterpret_cast<uint2*>(shared_scales + atom * kAtomStride + offset) =
        make_uint2(value.x, value.y);
    *reinterpret_cast<uint2*>(shared_scales + atom * kAtomStride + offset + 8) =
        make_uint2(value.z, value.w);
  }
  for (int index = threadIdx.x; index < kMaxTokens * kTileK; index += kThreads) {
    const int token = index / kTileK;
    const int offset = index % kTileK;
    const int source = k_begin + offset;
    __nv_bfloat16 value = __float2bfloat16_rn(0.0f);
    if (token < m && source < k) value = input[static_cast<size_t>(token) * k + source];
    shared_x[token * kTokenStride + (offset & ~31) + staged_position(offset & 31)] = value;
  }
  __syncthreads();

  // B fragments of this thread: token `group`, chunk `chunk`, 32 staged elements = 16 words.
  uint32_t b[16];
  {
    const uint4* source =
        reinterpret_cast<const uint4*>(shared_x + group * kTokenStride + chunk * 32);
#pragma unroll
    for (int part = 0; part < 4; ++part) {
      const uint4 value = source[part];
      b[part * 4 + 0] = value.x;
      b[part * 4 + 1] = value.y;
      b[part * 4 + 2] = value.z;
      b[part * 4 + 3] = value.w;
    }
  }

  const int scale_atom = chunk >> 1;
  const int scale_byte = (chunk & 1) * 2;
#pragma unroll
  for (int step = 0; step < 4; ++step) {
    float accumulator[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    uint32_t multiplier[2][2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row_in_tile = warp_rows * 64 + step * 16 + half * 8 + group;
      const uint16_t two = *reinterpret_cast<const uint16_t*>(
          shared_scales + scale_atom * kAtomStride + (row_in_tile & 31) * 16 +
          (row_in_tile >> 5) * 4 + scale_byte);
      multiplier[half][0] = scale_multiplier(static_cast<uint8_t>(two & 0xffu));
      multiplier[half][1] = scale_multiplier(static_cast<uint8_t>(two >> 8));
    }
    const uint32_t words[2][4] = {
        {packed[step][0].x, packed[step][0].y, packed[step][0].z, packed[step][0].w},
        {packed[step][1].x, packed[step][1].y, packed[step][1].z, packed[step][1].w}};
#pragma unroll
    for (int word = 0; word < 4; ++word) {
      uint32_t low[4], high[4];
      place_e2m1x8(words[0][word], low);    // row `group`
      place_e2m1x8(words[1][word], high);   // row `group + 8`
      const uint32_t scale_low = multiplier[0][word >> 1];
      const uint32_t scale_high = multiplier[1][word >> 1];
#pragma unroll
      for (int pair = 0; pair < 2; ++pair) {
        // One MMA: this thread's k-slots (2t, 2t+1) and (2t+8, 2t+9) are staged pairs
        // 2*pair and 2*pair+1 of the word, for both rows.
        mma_bf16_16x8x16(accumulator, mul_bf16x2(low[2 * pair], scale_low),
                         mul_bf16x2(high[2 * pair], scale_high),
                         mul_bf16x2(low[2 * pair + 1], scale_low),
                         mul_bf16x2(high[2 * pair + 1], scale_high), b[word * 4 + 2 * pair],
                         b[word * 4 + 2 * pair + 1]);
      }
    }
    // accumulator: rows (group, group + 8) x tokens (2*quad, 2*quad + 1)
    const int row_in_tile = warp_rows * 64 + step * 16 + group;
    *reinterpret_cast<float2*>(&shared_sums[warp_k][row_in_tile][2 * quad]) =
        make_float2(accumulator[0], accumulator[1]);
    *reinterpret_cast<float2*>(&shared_sums[warp_k][row_in_tile + 8][2 * quad]) =
        make_float2(accumulator[2], accumulator[3]);
  }
  __syncthreads();

  // 128 rows x 8 tokens: four threads... one (row, token pair-of-four) per thread.
  const float finish = global_scale * 256.0f;  // undo the 2^-8 left by the scale multiplier
  for (int index = threadIdx.x; index < kTileRows * kMaxTokens; index += kThreads) {
    const int row_in_tile = index / kMaxTokens;
    const int token = index % kMaxTokens;
    const float sum = (shared_sums[0][row_in_tile][token] + shared_sums[1][row_in_tile][token]) +
                      (shared_sums[2][row_in_tile][token] + shared_sums[3][row_in_tile][token]);
    const int row = row_tile * kTileRows + row_in_tile;
    if (slices == 1) {
      if (row < n && token < m) {
        output[static_cast<size_t>(token) * n + row] = __float2bfloat16_rn(sum * finish);
      }
    } else {
      partials[(static_cast<size_t>(slice) * gridDim.x * kTileRows + row) * kMaxTokens + token] =
          sum;
    }
  }
  if (slices == 1) return;

  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int arrived = atomicAdd(&counters[row_tile], 1u);
    last_arrival = arrived == static_cast<unsigned int>(slices - 1);
    if (last_arrival) counters[row_tile] = 0u;
  }
  __syncthreads();
  if (!last_arrival) return;
  __threadfence();
  for (int index = threadIdx.x; index < kTileRows * kMaxTokens; index += kThreads) {
    const int row_in_tile = index / kMaxTokens;
    const int token = index % kMaxTokens;
    const int row = row_tile * kTileRows + row_in_tile;
    float total = 0.0f;
    for (int part = 0; part < slices; ++part) {
      total += __ldcg(partials +
                      (static_cast<size_t>(part) * gridDim.x * kTileRows + row) * kMaxTokens + token);
    }
    if (row < n && token < m) {
      output[static_cast<size_t>(token) * n + row] = __float2bfloat16_rn(total * finish);
    }
  }
}

}  // namespace nvfp4_vector
}  // namespace mircuda_b200

extern "C" int mircuda_b200_nvfp4_vector_create(int m, int n, int k, void* stream,
                                                void** output) {
  using namespace mircuda_b200::nvfp4_vector;
  if (m <= 0 || m > kMaxTokens || n <= 0 || k <= 0 || k % 64 != 0 || stream == nullptr ||
      output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->m = m;
  plan->n = n;
  plan->k = k;
  plan->slices = (k + kTileK - 1) / kTileK;
  plan->stream = static_cast<cudaStream_t>(stream);
  const size_t row_tiles = (static_cast<size_t>(n) + kTileRows - 1) / kTileRows;
  int status = 0;
  if (plan->slices > 1) {
    status = static_cast<int>(cudaMallocAsync(
        reinterpret_cast<void**>(&plan->partials),
        static_cast<size_t>(plan->slices) * row_tiles * kTileRows * kMaxTokens * sizeof(float),
        plan->stream));
    if (status == 0) {
      status = static_cast<int>(cudaMallocAsync(reinterpret_cast<void**>(&plan->counters),
                                                row_tiles * sizeof(unsigned int), plan->stream));
    }
    if (status == 0) {
      status = static_cast<int>(
          cudaMemsetAsync(plan->counters, 0, row_tiles * sizeof(unsigned int), plan->stream));
    }
  }
  if (status != 0) {
    if (plan->partials != nullptr) cudaFreeAsync(plan->partials, plan->stream);
    if (plan->counters != nullptr) cudaFreeAsync(plan->counters, plan->stream);
    delete plan;
    return status;
  }
  *output = plan;
  return 0;
}

extern "C" int mircuda_b200_nvfp4_vector_execute(void* raw, void* stream, const void* input,
                                                 const void* weight, const void* weight_scales,
                                                 void* output, float global_scale) {
  using namespace mircuda_b200::nvfp4_vector;
  if (raw == nullptr || stream == nullptr || input == nullptr || weight == nullptr ||
      weight_scales == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(weight_scales)) & 15u) !=
      0u) {
    return -1;
  }
  const dim3 grid((plan->n + kTileRows - 1) / kTileRows, plan->slices);
  nvfp4_vector_kernel<<<grid, kThreads, 0, cuda_stream>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
      static_cast<const uint8_t*>(weight_scales), static_cast<__nv_bfloat16*>(output),
      plan->partials, plan->counters, plan->m, plan->n, plan->k, plan->slices, global_scale);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" void mircuda_b200_nvfp4_vector_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::nvfp4_vector::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->partials != nullptr) cudaFreeAsync(plan->partials, plan->stream);
  if (plan->counters != nullptr) cudaFreeAsync(plan->counters, plan->stream);
  delete plan;
}
