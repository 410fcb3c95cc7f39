// bf16 -> NVFP4 quantizer (E2M1 codes, one UE4M3 scale per 16 K-elements, per-tensor fp32
// global scale). The reference has no such quantizer; the rule implemented here is
//   global = amax_tensor / (448 * 6)              (1.0 for an all-zero tensor)
//   s_blk  = rne_ue4m3(amax_blk / (6 * global))
//   code   = rne_e2m1(x / (ue4m3(s_blk) * global)), saturating at +-6; 0 when s_blk == 0
// with every operation in round-to-nearest fp32. Conversions use the sm_100a cvt
// instructions. The kernel is bound by HBM: 2 bytes in, 0.5625 bytes out per element.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "fp4_codec.cuh"
#include "launch_overlap.hpp"
#include "layout.cuh"
#include "nvfp4_block.cuh"
#include "ptx.cuh"

namespace mircuda_b200 {
namespace {

using nvfp4_block::magnitude_bits;
using nvfp4_block::max_magnitude;
using nvfp4_block::quantize_block16;
using nvfp4_block::swiglu8;

// Largest |x| as bf16 magnitude bits, combined across the grid with an integer atomic max.
__global__ void __launch_bounds__(256)
nvfp4_amax_kernel(const uint4* __restrict__ input, size_t vectors, const uint16_t* __restrict__ tail,
            size_t tail_elements, unsigned int* __restrict__ result) {
  uint32_t maximum = 0u;
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < vectors;
       index += static_cast<size_t>(gridDim.x) * blockDim.x) {
    maximum = max(maximum, max_magnitude(__ldg(input + index)));
  }
  if (blockIdx.x == 0 && threadIdx.x < tail_elements) {
    maximum = max(maximum, magnitude_bits(tail[threadIdx.x]));
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    maximum = max(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
  }
  if ((threadIdx.x & 31) == 0 && maximum != 0u) atomicMax(result, maximum);
}

__global__ void nvfp4_finish_global_scale_kernel(unsigned int* word) {
  const uint32_t magnitude = *word;  // bf16 bits of the tensor amax
  const float amax = __uint_as_float(magnitude << 16);
  const float global = amax > 0.0f ? __fdiv_rn(amax, 2688.0f) : 1.0f;
  *reinterpret_cast<float*>(word) = global;
}

// One thread per 16-element block: two 16-byte loads, one 8-byte store, one scale byte.
// ROW_MAJOR_SCALES: scales go to [rows, k/16] bytes instead of the swizzled atoms, so that
// whole rows (codes and scales) can be moved to another place before the layout is fixed.
// SWIGLU: the input is [rows, 2k] (gate columns then up columns) and the quantised tensor is
// silu(gate) * up rounded to bf16, which is never written to memory.
template <bool ROW_MAJOR_SCALES, bool SWIGLU>
__global__ void __launch_bounds__(256)
nvfp4_quantize_kernel(const uint4* __restrict__ input, const float* __restrict__ global_scale,
                uint2* __restrict__ codes, uint8_t* __restrict__ scales, uint32_t rows,
                const unsigned int* __restrict__ row_bound, uint32_t k) {
  // Launched so that it may be scheduled while the kernel before it is finishing; nothing is
  // read before that kernel has completed.
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  if (row_bound != nullptr) rows = min(rows, __ldg(row_bound));
  const uint32_t blocks_per_row = k / 16u;
  const size_t block = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (block >= static_cast<size_t>(rows) * blocks_per_row) return;
  uint4 first, second;
  if (SWIGLU) {
    const size_t row_index = block / blocks_per_row;
    const size_t vector = row_index * (blocks_per_row * 4u) + (block - row_index * blocks_per_row) * 2u;
    const size_t up = vector + blocks_per_row * 2u;       // k / 8 sixteen-byte vectors further
    first = swiglu8(__ldg(input + vector), __ldg(input + up));
    second = swiglu8(__ldg(input + vector + 1u), __ldg(input + up + 1u));
  } else {
    first = __ldg(input + block * 2u);
    second = __ldg(input + block * 2u + 1u);
  }
  uint8_t scale_code = 0u;
  codes[block] = quantize_block16(first, second, *global_scale, &scale_code);
  const uint32_t row = static_cast<uint32_t>(block / blocks_per_row);
  const uint32_t column = static_cast<uint32_t>(block % blocks_per_row);
  scales[ROW_MAJOR_SCALES ? block : scale_offset(row, column, blocks_per_row)] = scale_code;
}

}  // namespace
}  // namespace mircuda_b200

extern "C" int mircuda_b200_nvfp4_global_scale(const void* input, size_t elements,
                                               void* global_scale, void* stream) {
  using namespace mircuda_b200;
  if (input == nullptr || global_scale == nullptr || stream == nullptr || elements == 0u) return -1;
  if ((reinterpret_cast<uintptr_t>(input) & 15u) != 0u ||
      (reinterpret_cast<uintptr_t>(global_scale) & 3u) != 0u) {
    return -1;
  }
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  int status = static_cast<int>(cudaMemsetAsync(global_scale, 0, sizeof(float), cuda_stream));
  if (status != 0) return status;
  const size_t vectors = elements / 8u;
  const size_t tail = elements % 8u;
  size_t blocks = (vectors + 255u) / 256u;
  if (blocks > 148u * 8u) blocks = 148u * 8u;
  if (blocks == 0u) blocks = 1u;
  nvfp4_amax_kernel<<<static_cast<unsigned int>(blocks), 256, 0, cuda_stream>>>(
      static_cast<const uint4*>(input), vectors,
      static_cast<const uint16_t*>(input) + vectors * 8u, tail,
      static_cast<unsigned int*>(global_scale));
  nvfp4_finish_global_scale_kernel<<<1, 1, 0, cuda_stream>>>(static_cast<unsigned int*>(global_scale));
  return static_cast<int>(cudaPeekAtLastError());
}

namespace mircuda_b200 {
namespace {

template <bool ROW_MAJOR_SCALES, bool SWIGLU = false>
int launch_quantize(const void* input, const void* global_scale, void* codes, void* scales,
                    uint32_t rows, uint32_t k, void* stream,
                    const unsigned int* row_bound = nullptr) {
  if (input == nullptr || global_scale == nullptr || codes == nullptr || scales == nullptr ||
      stream == nullptr || rows == 0u || k == 0u || k % 64u != 0u) {
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(input) & 15u) != 0u ||
      (reinterpret_cast<uintptr_t>(codes) & 7u) != 0u) {
    return -1;
  }
  const size_t blocks = static_cast<size_t>(rows) * (k / 16u);
  const size_t grid = (blocks + 255u) / 256u;
  if (grid > 0x7fffffffull) return -1;
  return launch_after_dependency(nvfp4_quantize_kernel<ROW_MAJOR_SCALES, SWIGLU>,
                                 dim3(static_cast<unsigned int>(grid)), dim3(256), 0,
                                 static_cast<cudaStream_t>(stream), static_cast<const uint4*>(input),
                                 static_cast<const float*>(global_scale), static_cast<uint2*>(codes),
                                 static_cast<uint8_t*>(scales), rows, row_bound, k);
}

}  // namespace
}  // namespace mircuda_b200

extern "C" int mircuda_b200_nvfp4_quantize_bf16(const void* input, const void* global_scale,
                                                void* codes, void* scales, uint32_t rows,
                                                uint32_t k, void* stream) {
  return mircuda_b200::launch_quantize<false>(input, global_scale, codes, scales, rows, k, stream);
}

extern "C" int mircuda_b200_nvfp4_quantize_rows_bf16(const void* input, const void* global_scale,
                                                     void* codes, void* row_scales, uint32_t rows,
                                                     uint32_t k, void* stream) {
  return mircuda_b200::launch_quantize<true>(input, global_scale, codes, row_scales, rows, k, stream);
}

extern "C" int mircuda_b200_moe_swiglu_nvfp4(const void* input, const void* global_scale,
                                             void* codes, void* scales, uint32_t rows,
                                             const unsigned int* row_bound, uint32_t intermediate,
                                             void* stream) {
  return mircuda_b200::launch_quantize<false, true>(input, global_scale, codes, scales, rows,
                                                    intermediate, stream, row_bound);
}
