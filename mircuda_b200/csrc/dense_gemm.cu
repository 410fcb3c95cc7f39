// Dense f16 / bf16 GEMM on sm_100a: C[M,N] = alpha * A[M,K] . B[N,K]^T + beta * C, fp32
// accumulation in tensor memory, output in the input type or fp32. Replaces the reference's
// CUTLASS dense plans (sys/native/dense_sm120.cu:130-184) behind the same C entry points, and
// is the tensor-core half of the int4 W4A16 path for M > 16 (w4a16_int4.cu).
//
// Aligned shapes (K and N multiples of 8) run the persistent tcgen05 tile kernel of
// dense_tile.cuh with kind::f16 and 128 x 256 tiles; this file supplies its epilogue (alpha,
// beta, conversion, row- and column-predicated stores). Other shapes take a plain CUDA-core
// kernel (they are tiny by construction: a row pitch that is not a multiple of 16 bytes cannot
// be described to TMA).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <new>

#include <cstdlib>

#include "dense_pair.cuh"
#include "dense_tile.cuh"
#include "ptx.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace dense_gemm {

using dense_tile::kBlockM;
using dense_tile::kThreads;
using dense_tile::Layout;
using dense_tile::dense_tile_kernel;

enum : int { kF16 = 0, kBf16 = 1, kF32 = 2 };

__device__ __forceinline__ float load_output(const void* c, size_t index, int type) {
  if (type == kF32) return static_cast<const float*>(c)[index];
  if (type == kBf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(c)[index]);
  return __half2float(static_cast<const __half*>(c)[index]);
}

__device__ __forceinline__ void store_output(void* c, size_t index, int type, float value) {
  if (type == kF32) {
    static_cast<float*>(c)[index] = value;
  } else if (type == kBf16) {
    static_cast<__nv_bfloat16*>(c)[index] = __float2bfloat16_rn(value);
  } else {
    static_cast<__half*>(c)[index] = __float2half_rn(value);
  }
}

// Warps 2-5 of the tile kernel call this with 32 consecutive accumulator columns of one row.
struct Epilogue {
  static constexpr uint32_t kElementBytes = 2u;
  void* c;
  int output_type;
  float alpha, beta;

  __device__ __forceinline__ void store(uint32_t row, uint32_t column, const uint32_t (&values)[32],
                                        uint32_t n) const {
    const size_t base = static_cast<size_t>(row) * n + column;
    if (output_type != kF32 && beta == 0.0f && column + 32u <= n) {
      // Two-byte outputs without a C operand: packed 16-byte stores (n % 8 == 0).
#pragma unroll
      for (uint32_t part = 0; part < 4u; ++part) {
        uint32_t packed[4];
#pragma unroll
        for (uint32_t pair = 0; pair < 4u; ++pair) {
          const float low = __uint_as_float(values[part * 8u + pair * 2u]) * alpha;
          const float high = __uint_as_float(values[part * 8u + pair * 2u + 1u]) * alpha;
          if (output_type == kBf16) {
            const __nv_bfloat162 two = __floats2bfloat162_rn(low, high);
            packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
          } else {
            const __half2 two = __floats2half2_rn(low, high);
            packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
          }
        }
        reinterpret_cast<uint4*>(static_cast<uint8_t*>(c) + base * 2u)[part] =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    } else {
#pragma unroll
      for (uint32_t item = 0; item < 32u; ++item) {
        if (column + item < n) {
          float value = __uint_as_float(values[item]) * alpha;
          if (beta != 0.0f) value = fmaf(beta, load_output(c, base + item, output_type), value);
          store_output(c, base + item, output_type, value);
        }
      }
    }
  }
};

// Shapes TMA cannot describe (K or N not a multiple of 8): one thread per output element.
__global__ void dense_gemm_plain_kernel(const void* __restrict__ a, const void* __restrict__ b,
                                        void* __restrict__ c, uint32_t m, uint32_t n, uint32_t k,
                                        int input_type, int output_type, float alpha, float beta) {
  const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= static_cast<size_t>(m) * n) return;
  const uint32_t row = static_cast<uint32_t>(index / n);
  const uint32_t column = static_cast<uint32_t>(index % n);
  float sum = 0.0f;
  for (uint32_t item = 0; item < k; ++item) {
    sum = fmaf(load_output(a, static_cast<size_t>(row) * k + item, input_type),
               load_output(b, static_cast<size_t>(column) * k + item, input_type), sum);
  }
  float value = sum * alpha;
  if (beta != 0.0f) value = fmaf(beta, load_output(c, index, output_type), value);
  store_output(c, index, output_type, value);
}

struct Plan {
  int input_type, output_type;
  int m, n, k;
  int device, sm_count;
  bool aligned;
  cudaStream_t stream;
  uint32_t* status;          // pinned
  const void* cached_a;
  const void* cached_b;
  CUtensorMap map_a, map_b;
  bool pair;                 // more than 128 rows of A: CTA pairs (dense_pair.cuh)
  int resident_pairs;
};

constexpr uint32_t kBlockN = 256, kStages = 4, kAccStages = 2;
constexpr uint32_t kPairStages = 6;     // a CTA of a pair holds 32 KB per stage

int encode_operand(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k, uint32_t box_rows) {
  return encode_k_major_map(map, base, rows, k, 2u, box_rows);
}

}  // namespace dense_gemm
}  // namespace mircuda_b200

extern "C" int mircuda_dense_create(int input_type, int output_type, int m, int n, int k,
                                    void* stream, void** output) {
  using namespace mircuda_b200::dense_gemm;
  if ((input_type != kF16 && input_type != kBf16) ||
      (output_type != input_type && output_type != kF32) || m <= 0 || n <= 0 || k <= 0 ||
      stream == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->input_type = input_type;
  plan->output_type = output_type;
  plan->m = m;
  plan->n = n;
  plan->k = k;
  plan->aligned = k % 8 == 0 && n % 8 == 0;
  plan->stream = static_cast<cudaStream_t>(stream);
  int status = static_cast<int>(cudaGetDevice(&plan->device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&plan->sm_count,
                                                     cudaDevAttrMultiProcessorCount, plan->device));
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
  // More than 128 rows of A run on CTA pairs (MIRCUDA_B200_DENSE_PAIR=0 keeps single CTAs).
  const char* pair_choice = std::getenv("MIRCUDA_B200_DENSE_PAIR");
  plan->pair = plan->aligned && m > static_cast<int>(kBlockM) && !(pair_choice != nullptr && pair_choice[0] == '0');
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

extern "C" size_t mircuda_dense_workspace_bytes(const void*) { return 0; }

extern "C" int mircuda_dense_execute(void* raw, void* stream, const void* a, const void* b,
                                     void* c, float alpha, float beta) {
  using namespace mircuda_b200;
  using namespace mircuda_b200::dense_gemm;
  if (raw == nullptr || stream == nullptr || a == nullptr || b == nullptr || c == nullptr) return -1;
  auto* plan = static_cast<Plan*>(raw);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  const bool pointers_aligned =
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) == 0u;
  if (!plan->aligned || !pointers_aligned) {
    const size_t elements = static_cast<size_t>(plan->m) * plan->n;
    dense_gemm_plain_kernel<<<static_cast<unsigned int>((elements + 255) / 256), 256, 0, cuda_stream>>>(
        a, b, c, plan->m, plan->n, plan->k, plan->input_type, plan->output_type, alpha, beta);
    return static_cast<int>(cudaPeekAtLastError());
  }
  if (a != plan->cached_a) {
    const int status = encode_operand(&plan->map_a, a, plan->m, plan->k, kBlockM);
    if (status != 0) return status;
    plan->cached_a = a;
  }
  if (b != plan->cached_b) {
    const int status = encode_operand(&plan->map_b, b, plan->n, plan->k, plan->pair ? kBlockN / 2u : kBlockN);
    if (status != 0) return status;
    plan->cached_b = b;
  }
  if (plan->pair) {
    return mircuda_b200::dense_pair::launch<kBlockN, kPairStages, kAccStages, Epilogue>(
        cuda_stream, plan->resident_pairs, plan->map_a, plan->map_b, plan->m, plan->n, plan->k,
        ptx::make_f16_idesc(plan->input_type == kBf16, 2u * kBlockM, kBlockN),
        Epilogue{c, plan->output_type, alpha, beta}, plan->status);
  }
  const uint32_t tiles = ((plan->m + kBlockM - 1u) / kBlockM) * ((plan->n + kBlockN - 1u) / kBlockN);
  const uint32_t grid = tiles < static_cast<uint32_t>(plan->sm_count) ? tiles : plan->sm_count;
  const uint32_t idesc = ptx::make_f16_idesc(plan->input_type == kBf16, kBlockM, kBlockN);
  dense_tile_kernel<kBlockN, kStages, kAccStages, Epilogue>
      <<<grid, kThreads, Layout<kBlockN, kStages, kAccStages>::kDynamicBytes, cuda_stream>>>(
          plan->map_a, plan->map_b, plan->m, plan->n, plan->k, idesc,
          Epilogue{c, plan->output_type, alpha, beta}, plan->status);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" void mircuda_dense_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::dense_gemm::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
