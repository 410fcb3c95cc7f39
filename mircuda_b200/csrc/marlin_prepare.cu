// One-time weight preparation and per-step route bucketing for the Marlin-layout W4A16
// path. These are pure layout conversions (integer work, bit-exact by definition); they
// replace the reference's sys/native/marlin/repack.cu behind the same C entry points, and the
// byte layouts they produce are the ones the reference's tests pin
// (tests/marlin/main.rs:139-217, tests/marlin/padded.rs:127-203, tests/marlin/routes.rs).
//
// Packed 4-bit weights: per expert, tiles of 16 (k) x 64 (n) ordered k-tile major; a tile is
// 128 u32; word `lane * 4 + quarter` (lane 0..31, quarter 0..3) belongs to rows
// n = tile_n*64 + quarter*16 + lane/4 (and n + 8) and columns k = tile_k*16 + (lane%4)*2 +
// {0, 1, 8, 9}; its eight nibbles, low to high, are
//   (n,k) (n,k+8) (n+8,k) (n+8,k+8) (n,k+1) (n,k+9) (n+8,k+1) (n+8,k+9)
// i.e. exactly one thread's A fragment of mma.m16n8k16, arranged so that nibble pairs
// (p, p+4) are the fragment's register pairs. Group scales: logical index group*N + n,
// permuted inside every run of 64 so that one thread's eight scales are 8 adjacent bytes.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "fp4_codec.cuh"

namespace mircuda_b200 {
namespace marlin {

struct Source {
  const uint8_t* left;
  const uint8_t* right;      // second half of the rows (gate | up pair), or null
  int size_n, size_k;        // padded physical extents of the packed matrix
  int logical_n, logical_k;  // extents of the canonical source
  bool interleaved;          // source rows alternate gate, up; packed rows are gate..., up...
};

// Row of the canonical source that packed row n takes its data from, and which buffer;
// -1 when the packed row is padding.
__device__ __forceinline__ int source_row(const Source& s, int n, const uint8_t** buffer,
                                          int* rows_in_buffer) {
  *buffer = s.left;
  *rows_in_buffer = s.logical_n;
  if (s.interleaved) {
    const int half = s.size_n / 2;
    const bool up = n >= half;
    const int unit = up ? n - half : n;
    if (unit >= s.logical_n / 2) return -1;
    return unit * 2 + (up ? 1 : 0);
  }
  if (s.right != nullptr) {
    const int half = s.size_n / 2;
    *rows_in_buffer = s.logical_n / 2;
    if (n >= half) {
      *buffer = s.right;
      n -= half;
    }
    return n < *rows_in_buffer ? n : -1;
  }
  return n < s.logical_n ? n : -1;
}

__device__ __forceinline__ uint32_t source_nibble(const Source& s, int expert, int n, int k) {
  if (k >= s.logical_k) return 0u;
  const uint8_t* buffer;
  int rows;
  const int row = source_row(s, n, &buffer, &rows);
  if (row < 0) return 0u;
  const uint8_t byte =
      buffer[(static_cast<size_t>(expert) * rows + row) * (s.logical_k / 2) + k / 2];
  return (byte >> ((k & 1) * 4)) & 0xfu;
}

// One thread per packed word.
__global__ void __launch_bounds__(256)
marlin_repack_kernel(Source s, uint32_t* __restrict__ output, int experts) {
  const size_t words_per_expert = static_cast<size_t>(s.size_n) * s.size_k / 8;
  const size_t word = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (word >= words_per_expert * experts) return;
  const int expert = static_cast<int>(word / words_per_expert);
  const int in_expert = static_cast<int>(word % words_per_expert);
  const int tiles_n = s.size_n / 64;
  const int tile = in_expert / 128;
  const int in_tile = in_expert % 128;
  const int lane = in_tile / 4;
  const int quarter = in_tile % 4;
  const int n = (tile % tiles_n) * 64 + quarter * 16 + lane / 4;
  const int k = (tile / tiles_n) * 16 + (lane % 4) * 2;
  uint32_t packed = 0u;
#pragma unroll
  for (int position = 0; position < 8; ++position) {
    // position bits: 0 -> +8 columns, 1 -> +8 rows, 2 -> +1 column
    const int row = n + ((position >> 1) & 1) * 8;
    const int column = k + (position & 1) * 8 + ((position >> 2) & 1);
    packed |= source_nibble(s, expert, row, column) << (position * 4);
  }
  output[word] = packed;
}

// Destination of logical scale index `linear` (= group * N + n) inside its expert.
__device__ __forceinline__ int scale_destination(int linear) {
  const int local = linear & 63;
  const int permuted = 8 * (local & 7) + (local >> 3);
  const int in_quad = permuted & 3;
  const int swapped = in_quad == 1 ? 2 : (in_quad == 2 ? 1 : in_quad);
  return (linear & ~63) + (permuted & ~3) + swapped;
}

// E8M0 group-32 scales (MXFP4): permute, pad with 127 (= 1.0).
__global__ void __launch_bounds__(256)
marlin_mxfp4_scales_kernel(const uint8_t* __restrict__ input, uint8_t* __restrict__ output,
                           Source s, int experts) {
  const int groups = s.size_k / 32;
  const int per_expert = s.size_n * groups;
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= per_expert * experts) return;
  const int expert = index / per_expert;
  const int logical = index % per_expert;
  const int group = logical / s.size_n;
  const int n = logical % s.size_n;
  uint8_t value = 127u;
  if (group < s.logical_k / 32) {
    const uint8_t* buffer;
    int rows;
    const int row = source_row(s, n, &buffer, &rows);
    if (row >= 0) {
      value = input[(static_cast<size_t>(expert) * s.logical_n + row) * (s.logical_k / 32) + group];
    }
  }
  output[static_cast<size_t>(expert) * per_expert + scale_destination(logical)] = value;
}

__global__ void __launch_bounds__(256)
marlin_scale_maximum_kernel(const uint8_t* __restrict__ left, const uint8_t* __restrict__ right,
                            unsigned int* __restrict__ maximum, int elements) {
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  float value = 0.0f;
  if (index < elements) {
    value = decode_e4m3_signed(left[index]);
    if (right != nullptr) value = fmaxf(value, decode_e4m3_signed(right[index]));
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
  }
  // Non-negative floats order like their bit patterns.
  if ((threadIdx.x & 31) == 0 && value > 0.0f) atomicMax(maximum, __float_as_uint(value));
}

// UE4M3 group-16 scales (NVFP4) -> the 8-bit "5 exponent + 3 mantissa bits of an f16" code the
// Marlin kernels read, after scaling the whole tensor by the largest power of two that keeps
// max_scale * 128 * factor below 57344; values that would fall below 2.0 become 0. The
// per-expert global scales absorb 2^119 / factor.
__global__ void __launch_bounds__(256)
marlin_nvfp4_scales_kernel(const uint8_t* __restrict__ left, const uint8_t* __restrict__ right,
                           const float* __restrict__ globals, uint8_t* __restrict__ output,
                           float* __restrict__ output_globals,
                           const unsigned int* __restrict__ maximum, int experts, int size_n,
                           int size_k) {
  const int groups = size_k / 16;
  const int per_expert = size_n * groups;
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  const float scaled_maximum = __uint_as_float(*maximum) * 128.0f;
  const float factor = scaled_maximum > 0.0f && scaled_maximum < 57344.0f
                           ? exp2f(floorf(log2f(57344.0f / scaled_maximum)))
                           : 1.0f;
  if (index < per_expert * experts) {
    const int expert = index / per_expert;
    const int logical = index % per_expert;
    const int group = logical / size_n;
    int n = logical % size_n;
    const uint8_t* source = left;
    int source_n = size_n;
    if (right != nullptr) {
      source_n = size_n / 2;
      if (n >= source_n) {
        source = right;
        n -= source_n;
      }
    }
    const float value =
        decode_e4m3_signed(source[(static_cast<size_t>(expert) * source_n + n) * groups + group]);
    const __half scaled = __hmul(__float2half_rn(value * factor), __float2half_rn(128.0f));
    const uint16_t bits = __half_as_ushort(scaled);
    const uint8_t code =
        __half2float(scaled) < 2.0f ? 0u : static_cast<uint8_t>((bits >> 7) & 0xffu);
    output[static_cast<size_t>(expert) * per_expert + scale_destination(logical)] = code;
  }
  if (index < experts) output_globals[index] = globals[index] * exp2f(119.0f) / factor;
}

// Route bucketing in one CTA: count rows per expert, lay experts out in blocks of
// `block_size` rows, place each assignment in its expert's range, then order every expert's
// rows by assignment id so that results do not depend on scheduling. Unused slots of
// `sorted` hold `assignments` (the padding marker).
__global__ void __launch_bounds__(1024)
marlin_routes_kernel(const uint32_t* __restrict__ selected,
                     const __nv_bfloat16* __restrict__ routing, int32_t* __restrict__ sorted,
                     int32_t* __restrict__ expert_ids, int32_t* __restrict__ padded,
                     int32_t* __restrict__ offsets, float* __restrict__ routing_f32,
                     int assignments, int experts, int block_size) {
  extern __shared__ int32_t shared[];
  int32_t* counts = shared;
  int32_t* cursors = shared + experts;
  const int capacity = assignments + experts * (block_size - 1);
  for (int expert = threadIdx.x; expert < experts; expert += blockDim.x) counts[expert] = 0;
  for (int slot = threadIdx.x; slot < capacity; slot += blockDim.x) sorted[slot] = assignments;
  __syncthreads();
  for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
    const uint32_t expert = selected[a];
    if (expert < static_cast<uint32_t>(experts)) atomicAdd(&counts[expert], 1);
    routing_f32[a] = __bfloat162float(routing[a]);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int offset = 0;
    for (int expert = 0; expert < experts; ++expert) {
      offsets[expert] = offset;
      cursors[expert] = 0;
      const int blocks = (counts[expert] + block_size - 1) / block_size;
      for (int block = 0; block < blocks; ++block) expert_ids[offset / block_size + block] = expert;
      offset += blocks * block_size;
    }
    padded[0] = offset;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
    const uint32_t expert = selected[a];
    if (expert >= static_cast<uint32_t>(experts)) continue;
    const int rank = atomicAdd(&cursors[expert], 1);
    sorted[offsets[expert] + rank] = a;
  }
  __syncthreads();
  // Each expert's rows by increasing assignment id (they arrive almost ordered).
  for (int expert = threadIdx.x; expert < experts; expert += blockDim.x) {
    int32_t* rows = sorted + offsets[expert];
    const int count = counts[expert];
    for (int index = 1; index < count; ++index) {
      const int32_t row = rows[index];
      int position = index;
      while (position > 0 && rows[position - 1] > row) {
        rows[position] = rows[position - 1];
        --position;
      }
      rows[position] = row;
    }
  }
}

int launch_repack(void* stream, const Source& source, void* output, int experts) {
  if (stream == nullptr || source.left == nullptr || output == nullptr || experts <= 0 ||
      source.size_n <= 0 || source.size_k <= 0 || source.size_n % 64 != 0 ||
      source.size_k % 16 != 0) {
    return -1;
  }
  const size_t words = static_cast<size_t>(experts) * source.size_n * source.size_k / 8;
  const size_t blocks = (words + 255) / 256;
  if (blocks > 0x7fffffffull) return -1;
  marlin_repack_kernel<<<static_cast<unsigned int>(blocks), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(
      source, static_cast<uint32_t*>(output), experts);
  return static_cast<int>(cudaPeekAtLastError());
}

}  // namespace marlin
}  // namespace mircuda_b200

extern "C" int mircuda_marlin_nvfp4_repack(void* stream, const void* input, void* output,
                                           int experts, int size_n, int size_k) {
  using namespace mircuda_b200::marlin;
  const Source source{static_cast<const uint8_t*>(input), nullptr, size_n, size_k, size_n, size_k,
                      false};
  return launch_repack(stream, source, output, experts);
}

extern "C" int mircuda_marlin_nvfp4_repack_pair(void* stream, const void* left, const void* right,
                                                void* output, int experts, int size_n,
                                                int size_k) {
  using namespace mircuda_b200::marlin;
  if (right == nullptr) return -1;
  const Source source{static_cast<const uint8_t*>(left), static_cast<const uint8_t*>(right), size_n,
                      size_k, size_n, size_k, false};
  return launch_repack(stream, source, output, experts);
}

extern "C" int mircuda_marlin_mxfp4_repack(void* stream, const void* input, void* output,
                                           int experts, int size_n, int size_k, int logical_n,
                                           int logical_k, bool interleaved_gate_up) {
  using namespace mircuda_b200::marlin;
  if (logical_n <= 0 || logical_k <= 0 || logical_n > size_n || logical_k > size_k ||
      logical_k % 2 != 0) {
    return -1;
  }
  const Source source{static_cast<const uint8_t*>(input), nullptr, size_n, size_k, logical_n,
                      logical_k, interleaved_gate_up};
  return launch_repack(stream, source, output, experts);
}

extern "C" int mircuda_marlin_mxfp4_prepare_scales(void* stream, const void* input, void* output,
                                                   int experts, int size_n, int size_k,
                                                   int logical_n, int logical_k,
                                                   bool interleaved_gate_up) {
  using namespace mircuda_b200::marlin;
  if (stream == nullptr || input == nullptr || output == nullptr || experts <= 0 || size_n <= 0 ||
      size_k <= 0 || size_n % 64 != 0 || size_k % 32 != 0 || logical_n <= 0 || logical_k <= 0 ||
      logical_n > size_n || logical_k > size_k || logical_k % 32 != 0) {
    return -1;
  }
  const Source source{static_cast<const uint8_t*>(input), nullptr, size_n, size_k, logical_n,
                      logical_k, interleaved_gate_up};
  const size_t elements = static_cast<size_t>(experts) * size_n * (size_k / 32);
  if (elements > 0x7fffffffull) return -1;
  marlin_mxfp4_scales_kernel<<<static_cast<unsigned int>((elements + 255) / 256), 256, 0,
                               static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(input), static_cast<uint8_t*>(output), source, experts);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" int mircuda_marlin_nvfp4_prepare_scales(void* stream, const void* left,
                                                   const void* right, const void* globals,
                                                   void* output, void* output_globals,
                                                   void* maximum, int experts, int size_n,
                                                   int size_k) {
  using namespace mircuda_b200::marlin;
  if (stream == nullptr || left == nullptr || globals == nullptr || output == nullptr ||
      output_globals == nullptr || maximum == nullptr || experts <= 0 || size_n <= 0 ||
      size_k <= 0 || size_n % 64 != 0 || size_k % 16 != 0) {
    return -1;
  }
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  int status = static_cast<int>(cudaMemsetAsync(maximum, 0, sizeof(unsigned int), cuda_stream));
  if (status != 0) return status;
  const size_t input_elements =
      static_cast<size_t>(experts) * (right == nullptr ? size_n : size_n / 2) * (size_k / 16);
  const size_t output_elements = static_cast<size_t>(experts) * size_n * (size_k / 16);
  if (output_elements > 0x7fffffffull) return -1;
  marlin_scale_maximum_kernel<<<static_cast<unsigned int>((input_elements + 255) / 256), 256, 0,
                                cuda_stream>>>(
      static_cast<const uint8_t*>(left), static_cast<const uint8_t*>(right),
      static_cast<unsigned int*>(maximum), static_cast<int>(input_elements));
  size_t threads_needed = output_elements > static_cast<size_t>(experts) ? output_elements
                                                                        : static_cast<size_t>(experts);
  marlin_nvfp4_scales_kernel<<<static_cast<unsigned int>((threads_needed + 255) / 256), 256, 0,
                               cuda_stream>>>(
      static_cast<const uint8_t*>(left), static_cast<const uint8_t*>(right),
      static_cast<const float*>(globals), static_cast<uint8_t*>(output),
      static_cast<float*>(output_globals), static_cast<const unsigned int*>(maximum), experts,
      size_n, size_k);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" int mircuda_marlin_prepare_moe_routes(void* stream, const void* selected,
                                                 const void* routing, void* sorted,
                                                 void* expert_ids, void* padded, void* offsets,
                                                 void* routing_f32, int assignments, int experts,
                                                 int block_size) {
  using namespace mircuda_b200::marlin;
  if (stream == nullptr || selected == nullptr || routing == nullptr || sorted == nullptr ||
      expert_ids == nullptr || padded == nullptr || offsets == nullptr ||
      routing_f32 == nullptr || assignments <= 0 || experts <= 0 || block_size <= 0 ||
      static_cast<size_t>(experts) * 2 * sizeof(int32_t) > 48 * 1024) {
    return -1;
  }
  marlin_routes_kernel<<<1, 1024, static_cast<size_t>(experts) * 2 * sizeof(int32_t),
                         static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(selected), static_cast<const __nv_bfloat16*>(routing),
      static_cast<int32_t*>(sorted), static_cast<int32_t*>(expert_ids),
      static_cast<int32_t*>(padded), static_cast<int32_t*>(offsets),
      static_cast<float*>(routing_f32), assignments, experts, block_size);
  return static_cast<int>(cudaPeekAtLastError());
}
