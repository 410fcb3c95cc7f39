// FP4 x FP4 GEMV for decode (M = 1): y[N] = bf16(alpha * sum_blocks dot16 * sx * sw), E2M1
// codes two per byte (even k in the low nibble), one UE4M3 scale per 16 K-elements in the
// 128x4-swizzled layout. Replaces sys/native/fp4_vector_sm120.cu behind the same C entry
// points; numerics follow that kernel (each 16-wide dot is formed exactly, then scaled by
// the product of the two block scales and accumulated in fp32).
//
// Three kernels sit behind the plan: shapes with n % 128 == 0 and k % 2048 == 0 run on the
// streaming kernel of nvfp4_stream.cu (the activation vector dequantised into its MMA fragments;
// MIRCUDA_B200_FP4_VECTOR=stream, the default there), fp4_vector_tc.cu is the tcgen05 kernel
// (=tensor) and the CUDA-core kernel of this file (=simt) serves every other shape and the
// allocation-free entry point.
//
// The op streams 0.5625*N*K bytes once and is bound by HBM. Work is cut into tiles of
// 128 rows (one scale row-tile) by 512 K-elements (eight whole 512-byte scale atoms), one CTA
// per tile, so that every weight byte arrives through 16-byte loads with all of a tile's
// loads in flight at once, every scale atom is fetched whole and coalesced, and there are
// enough CTAs to fill the machine even for N = 4096. The activation slice a thread needs is
// the same for all its rows, so it is decoded to f16x2 registers once. Products of two E2M1
// values and sums of eight of them are exact in f16, so the inner loop is packed HFMA2.
// K-slices of one row tile meet in a scratch array of per-slice partial sums; the CTA that
// arrives last (a counter per row tile, no spinning) adds them in a fixed order, applies
// alpha and writes bf16, which keeps results deterministic.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <mutex>
#include <new>

#include <cstdlib>
#include <cstring>

#include "fp4_codec.cuh"
#include "fp4_vector_tc.hpp"
#include "nvfp4_stream.hpp"
#include "ptx.cuh"
#include "layout.cuh"

namespace mircuda_b200 {
namespace fp4_vector {

constexpr int kThreads = 256;
constexpr int kTileRows = 128;
constexpr int kTileK = 512;                       // elements per K-slice
constexpr int kAtomsPerTile = kTileK / 64;        // scale atoms (4 columns of 16) per slice
constexpr int kAtomStride = 512 + 8;              // padded in shared memory against bank conflicts
constexpr int kRowSteps = kTileRows / (kThreads / 16);

struct Plan {
  int n;
  int k;
  int slices;
  cudaStream_t stream;
  float* partials;          // [slices][row_tiles * 128]
  unsigned int* counters;   // [row_tiles], zero between launches
  fp4_vector_tc::Plan* tensor;   // the tensor-core implementation, when the plan uses it
  bool stream_kernel;            // the persistent streaming kernel of nvfp4_stream.cu
  bool overlap_launches;
  nvfp4_stream::Config stream_config;
  uint32_t* status;              // pinned; raised by a streaming launch whose bounded wait ran out
};

__global__ void __launch_bounds__(kThreads)
fp4_vector_kernel(const uint8_t* __restrict__ input, const uint8_t* __restrict__ input_scales,
       const uint8_t* __restrict__ weight, const uint8_t* __restrict__ weight_scales,
       __nv_bfloat16* __restrict__ output, float* __restrict__ partials,
       unsigned int* __restrict__ counters, int n, int k, int slices, float alpha) {
  __shared__ __align__(16) uint8_t shared_scales[kAtomsPerTile * kAtomStride];
  __shared__ bool last_arrival;

  const int row_tile = blockIdx.x;
  const int slice = blockIdx.y;
  const int k_begin = slice * kTileK;
  const int atoms_k = k / 64;
  const int lane16 = threadIdx.x & 15;
  const int row_group = threadIdx.x >> 4;          // 0..15
  const int element = k_begin + lane16 * 32;       // first of this thread's 32 K-elements
  const bool active = element < k;

  // Issue every weight load of the tile first: 8 x 16 bytes in flight per thread.
  uint4 packed[kRowSteps];
#pragma unroll
  for (int step = 0; step < kRowSteps; ++step) {
    const int row = row_tile * kTileRows + step * 16 + row_group;
    packed[step] = make_uint4(0u, 0u, 0u, 0u);
    if (active && row < n) {
      packed[step] = load_streaming_16(weight + (static_cast<size_t>(row) * k + element) / 2);
    }
  }

  // Whole scale atoms of this tile, coalesced: 8 atoms x 512 bytes = 256 threads x 16 bytes.
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

  // This thread's 32 activations (16 bytes) as f16x2 and their two block scales.
  __half2 x[16];
  float x_scale[2] = {0.0f, 0.0f};
  if (active) {
    const uint4 codes = __ldg(reinterpret_cast<const uint4*>(input + element / 2));
    decode_e2m1x32(codes, x);
    const int column = element / 16;
    const uint16_t two = *reinterpret_cast<const uint16_t*>(
        input_scales + scale_offset(0u, static_cast<uint32_t>(column), static_cast<uint32_t>(k / 16)));
    x_scale[0] = decode_ue4m3(static_cast<uint8_t>(two & 0xffu));
    x_scale[1] = decode_ue4m3(static_cast<uint8_t>(two >> 8));
  } else {
#pragma unroll
    for (int pair = 0; pair < 16; ++pair) x[pair] = __float2half2_rn(0.0f);
  }
  __syncthreads();

  const int scale_atom = lane16 >> 1;               // 64 elements per atom column group
  const int scale_byte = (lane16 & 1) * 2;          // two of its four columns
#pragma unroll
  for (int step = 0; step < kRowSteps; ++step) {
    const int row_in_tile = step * 16 + row_group;
    __half2 w[16];
    decode_e2m1x32(packed[step], w);
    float sum = 0.0f;
#pragma unroll
    for (int block = 0; block < 2; ++block) {
      __half2 dot = __float2half2_rn(0.0f);
#pragma unroll
      for (int pair = 0; pair < 8; ++pair) dot = __hfma2(x[block * 8 + pair], w[block * 8 + pair], dot);
      const uint8_t code = shared_scales[scale_atom * kAtomStride + (row_in_tile & 31) * 16 +
                                         (row_in_tile >> 5) * 4 + scale_byte + block];
      const float2 halves = __half22float2(dot);
      sum = fmaf(halves.x + halves.y, x_scale[block] * decode_ue4m3(code), sum);
    }
#pragma unroll
    for (int offset = 8; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
    if (lane16 == 0) {
      const int row = row_tile * kTileRows + row_in_tile;
      if (slices == 1) {
        if (row < n) output[row] = __float2bfloat16_rn(sum * alpha);
      } else {
        partials[static_cast<size_t>(slice) * gridDim.x * kTileRows + row] = sum;
      }
    }
  }
  if (slices == 1) return;

  // Last-arriving slice of this row tile reduces in slice order. No CTA waits on another.
  ptx::fence_acq_rel_gpu();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int arrived = atomicAdd(&counters[row_tile], 1u);
    last_arrival = arrived == static_cast<unsigned int>(slices - 1);
    if (last_arrival) counters[row_tile] = 0u;
  }
  __syncthreads();
  if (!last_arrival) return;
  ptx::fence_acq_rel_gpu();
  if (threadIdx.x < kTileRows) {
    const int row = row_tile * kTileRows + threadIdx.x;
    float total = 0.0f;
    for (int part = 0; part < slices; ++part) {
      total += __ldcg(partials + static_cast<size_t>(part) * gridDim.x * kTileRows + row);
    }
    if (row < n) output[row] = __float2bfloat16_rn(total * alpha);
  }
}

}  // namespace fp4_vector
}  // namespace mircuda_b200

extern "C" int mircuda_fp4_vector_create(int n, int k, void* stream, void** output) {
  using namespace mircuda_b200::fp4_vector;
  if (n <= 0 || k <= 0 || k % 64 != 0 || stream == nullptr || output == nullptr) return -1;
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->n = n;
  plan->k = k;
  plan->slices = (k + kTileK - 1) / kTileK;
  plan->stream = static_cast<cudaStream_t>(stream);
  // Two implementations. The tensor-core kernel (fp4_vector_tc.cu) streams faster but pays
  // about 2 us more per launch (tensor-memory allocation, pipeline fill, hand-over of K parts
  // through global memory); measured on B200 it wins from about 24 MB of weights up (0.59 of
  // HBM speed against 0.48 at 24576 x 4096, 0.17 against 0.22 at 4096 x 4096).
  // MIRCUDA_B200_FP4_VECTOR=tensor or =simt overrides the choice.
  // A third one, the persistent streaming kernel (nvfp4_stream.cu, shared with the bf16 x NVFP4
  // op: the activation vector is dequantised into the warps' MMA fragments once per launch),
  // beats both wherever it applies (whole 128-row scale tiles, K a multiple of 2048) and is the
  // default there; =stream, =tensor or =simt in MIRCUDA_B200_FP4_VECTOR force a choice.
  const char* choice = std::getenv("MIRCUDA_B200_FP4_VECTOR");
  const bool forced_other = choice != nullptr && (std::strcmp(choice, "tensor") == 0 || std::strcmp(choice, "simt") == 0);
  if (!forced_other && mircuda_b200::nvfp4_stream::eligible(n, k)) {
    int status = mircuda_b200::nvfp4_stream::prepare(&plan->stream_config, n, k);
    if (status == 0) {
      status = static_cast<int>(cudaHostAlloc(reinterpret_cast<void**>(&plan->status), sizeof(uint32_t),
                                              cudaHostAllocMapped));
      if (status != 0) {
        delete plan;
        return status;
      }
      *plan->status = 0u;
      plan->stream_kernel = true;
      // Overlapped launches (see mircuda_b200_nvfp4_vector_*): on unless the environment says 0.
      const char* overlap = std::getenv("MIRCUDA_B200_OVERLAP_LAUNCHES");
      plan->overlap_launches = overlap == nullptr || overlap[0] == '1';
      *output = plan;
      return 0;
    }
    if (status != -1) {
      delete plan;
      return status;
    }
  }
  bool tensor = static_cast<size_t>(n) * static_cast<size_t>(k) / 2u >= (size_t{24} << 20);
  if (choice != nullptr && std::strcmp(choice, "tensor") == 0) tensor = true;
  if (choice != nullptr && std::strcmp(choice, "simt") == 0) tensor = false;
  if (tensor) {
    const int status = mircuda_b200::fp4_vector_tc::create(n, k, plan->stream, &plan->tensor);
    if (status != 0) {
      delete plan;
      return status;
    }
    *output = plan;
    return 0;
  }
  const size_t row_tiles = (static_cast<size_t>(n) + kTileRows - 1) / kTileRows;
  int status = 0;
  if (plan->slices > 1) {
    status = static_cast<int>(cudaMallocAsync(
        reinterpret_cast<void**>(&plan->partials),
        static_cast<size_t>(plan->slices) * row_tiles * kTileRows * sizeof(float), plan->stream));
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

extern "C" int mircuda_fp4_vector_execute(void* raw, void* stream, const void* input,
                                          const void* input_scales, const void* weight,
                                          const void* weight_scales, void* output, float alpha) {
  using namespace mircuda_b200::fp4_vector;
  if (raw == nullptr || stream == nullptr || input == nullptr || input_scales == nullptr ||
      weight == nullptr || weight_scales == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight) |
        reinterpret_cast<uintptr_t>(weight_scales)) & 15u) != 0u) {
    return -1;
  }
  if (plan->stream_kernel) {
    if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
    if ((reinterpret_cast<uintptr_t>(input_scales) & 1u) != 0u) return -1;
    return mircuda_b200::nvfp4_stream::launch(&plan->stream_config, cuda_stream, plan->overlap_launches, input,
                                              input_scales, weight, weight_scales, output, 1, plan->n, plan->k,
                                              alpha, plan->status);
  }
  if (plan->tensor != nullptr) {
    if ((reinterpret_cast<uintptr_t>(input_scales) & 15u) != 0u) return -1;
    return mircuda_b200::fp4_vector_tc::execute(plan->tensor, cuda_stream, input, input_scales, weight,
                                                weight_scales, output, alpha);
  }
  const dim3 grid((plan->n + kTileRows - 1) / kTileRows, plan->slices);
  fp4_vector_kernel<<<grid, kThreads, 0, cuda_stream>>>(
      static_cast<const uint8_t*>(input), static_cast<const uint8_t*>(input_scales),
      static_cast<const uint8_t*>(weight), static_cast<const uint8_t*>(weight_scales),
      static_cast<__nv_bfloat16*>(output), plan->partials, plan->counters, plan->n, plan->k,
      plan->slices, alpha);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" void mircuda_fp4_vector_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::fp4_vector::Plan*>(raw);
  if (plan == nullptr) return;
  mircuda_b200::fp4_vector_tc::destroy(plan->tensor);
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  if (plan->partials != nullptr) cudaFreeAsync(plan->partials, plan->stream);
  if (plan->counters != nullptr) cudaFreeAsync(plan->counters, plan->stream);
  delete plan;
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some hosts may not let this library call the CUDA allocator at all: a serving process that
// handed every byte of device memory to its own arena at start-up (a later cudaMalloc would
// fail or evict), or a caller that only owns raw pointers inside somebody else's memory pool
// and must not grow the process footprint behind that pool's back. The plan-based entry
// points above allocate their cross-slice scratch with cudaMallocAsync when the plan is
// created; the entry point below needs no plan and no allocation. Its scratch lives in the two
// file-scope device arrays that follow, which every GPU that loads this library holds until
// the process exits (1 MiB + 4 KiB per device).
namespace mircuda_b200 {
namespace fp4_vector {

constexpr size_t kStaticPartialFloats = 262144;   // slices * padded rows must fit: 1 MiB
constexpr size_t kStaticRowTiles = 1024;          // N <= 131072

static __device__ __align__(256) float static_partials[kStaticPartialFloats];
static __device__ __align__(256) unsigned int static_counters[kStaticRowTiles];

struct StaticScratch {
  float* partials;
  unsigned int* counters;
  bool ready;
};

// In host code the array names above are host-side stand-ins, not device addresses; the
// device addresses are looked up once per device, with that device current, and cached.
int static_scratch(StaticScratch** result) {
  constexpr int kMaxDevices = 64;
  static StaticScratch cache[kMaxDevices] = {};
  static std::mutex guard;
  int device = 0;
  int status = static_cast<int>(cudaGetDevice(&device));
  if (status != 0) return status;
  if (device < 0 || device >= kMaxDevices) return -1;
  std::lock_guard<std::mutex> lock(guard);
  StaticScratch& entry = cache[device];
  if (!entry.ready) {
    void* partials = nullptr;
    void* counters = nullptr;
    status = static_cast<int>(cudaGetSymbolAddress(&partials, static_partials));
    if (status != 0) return status;
    status = static_cast<int>(cudaGetSymbolAddress(&counters, static_counters));
    if (status != 0) return status;
    entry.partials = static_cast<float*>(partials);
    entry.counters = static_cast<unsigned int*>(counters);
    entry.ready = true;
  }
  *result = &entry;
  return 0;
}

}  // namespace fp4_vector
}  // namespace mircuda_b200

extern "C" int mircuda_b200_fp4_vector_execute_static(int n, int k, void* stream,
                                                      const void* input,
                                                      const void* input_scales,
                                                      const void* weight,
                                                      const void* weight_scales, void* output,
                                                      float alpha) {
  using namespace mircuda_b200::fp4_vector;
  if (n <= 0 || k <= 0 || k % 64 != 0 || stream == nullptr || input == nullptr ||
      input_scales == nullptr || weight == nullptr || weight_scales == nullptr ||
      output == nullptr) {
    return -1;
  }
  if (((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weight) |
        reinterpret_cast<uintptr_t>(weight_scales)) & 15u) != 0u) {
    return -1;
  }
  const size_t slices = (static_cast<size_t>(k) + kTileK - 1) / kTileK;
  const size_t row_tiles = (static_cast<size_t>(n) + kTileRows - 1) / kTileRows;
  if (row_tiles > kStaticRowTiles || slices * row_tiles * kTileRows > kStaticPartialFloats) {
    return -4;  // the shape needs more scratch than the static arrays hold
  }
  StaticScratch* scratch = nullptr;
  int status = static_scratch(&scratch);
  if (status != 0) return status;
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (slices > 1) {
    // The arrays keep whatever the previous call left; the arrival counters must start at 0.
    status = static_cast<int>(cudaMemsetAsync(scratch->counters, 0,
                                              row_tiles * sizeof(unsigned int), cuda_stream));
    if (status != 0) return status;
  }
  const dim3 grid(static_cast<unsigned int>(row_tiles), static_cast<unsigned int>(slices));
  fp4_vector_kernel<<<grid, kThreads, 0, cuda_stream>>>(
      static_cast<const uint8_t*>(input), static_cast<const uint8_t*>(input_scales),
      static_cast<const uint8_t*>(weight), static_cast<const uint8_t*>(weight_scales),
      static_cast<__nv_bfloat16*>(output), scratch->partials, scratch->counters, n, k,
      static_cast<int>(slices), alpha);
  return static_cast<int>(cudaPeekAtLastError());
}
