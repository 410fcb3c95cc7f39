// Dense f16 / bf16 GEMM on sm_100a: C[M,N] = alpha * A[M,K] . B[N,K]^T + beta * C, fp32
// accumulation in tensor memory, output in the input type or fp32. Replaces the reference's
// CUTLASS dense plans (sys/native/dense_sm120.cu:130-184) behind the same C entry points, and
// is the tensor-core half of the int4 W4A16 path for M > 16 (w4a16_int4.cu).
//
// Aligned shapes (K and N multiples of 8) run a persistent tcgen05 kernel with the anatomy of
// the grouped kernels: one 192-thread CTA per SM, warp 0 issues TMA loads of 128-byte-swizzled
// K-major tiles (A 128 x 64, B BN x 64 elements per stage), warp 1 issues four
// tcgen05.mma.kind::f16 per stage, warps 2-5 drain the accumulator (alpha, beta, conversion,
// row- and column-predicated stores). Tiles are walked M-fastest so that CTAs running together
// share B tiles. Other shapes take a plain CUDA-core kernel (they are tiny by construction:
// a row pitch that is not a multiple of 16 bytes cannot be described to TMA).
// Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <new>

#include "ptx.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace dense_gemm {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kBlockKBytes = 128;     // 64 two-byte elements per stage row
constexpr uint32_t kBlockK = 64;
constexpr uint32_t kThreads = 192;
constexpr uint32_t kTmemColumns = 512;

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
struct Layout {
  static constexpr uint32_t kABytes = kBlockM * kBlockKBytes;
  static constexpr uint32_t kBBytes = BN * kBlockKBytes;
  static constexpr uint32_t kBOffset = STAGES * kABytes;
  static constexpr uint32_t kBarrierOffset = kBOffset + STAGES * kBBytes;
  static constexpr uint32_t kBarriers = 2 * STAGES + 2 * ACC_STAGES;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  static constexpr uint32_t kDynamicBytes = kMiscOffset + 16 + 1024;
  static_assert(ACC_STAGES * BN <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

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

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
__global__ void __launch_bounds__(kThreads, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  void* __restrict__ c, uint32_t m, uint32_t n, uint32_t k, int input_type,
                  int output_type, float alpha, float beta, uint32_t* __restrict__ status) {
  using L = Layout<BN, STAGES, ACC_STAGES>;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_a = shared;
  uint8_t* shared_b = shared + L::kBOffset;
  uint64_t* full = reinterpret_cast<uint64_t*>(shared + L::kBarrierOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(shared + L::kMiscOffset);
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const uint32_t warp = threadIdx.x / 32u;
  const uint32_t lane = threadIdx.x % 32u;

  if (threadIdx.x == 0) {
    for (uint32_t stage = 0; stage < STAGES; ++stage) {
      ptx::mbarrier_init(&full[stage], 1);
      ptx::mbarrier_init(&empty[stage], 1);
    }
    for (uint32_t stage = 0; stage < ACC_STAGES; ++stage) {
      ptx::mbarrier_init(&acc_full[stage], 1);
      ptx::mbarrier_init(&acc_empty[stage], 4);
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&map_a);
    ptx::prefetch_tensor_map(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_allocate(tmem_slot, kTmemColumns);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t tiles_m = (m + kBlockM - 1u) / kBlockM;
  const uint32_t tiles_n = (n + BN - 1u) / BN;
  const uint32_t tiles = tiles_m * tiles_n;
  const uint32_t k_tiles = (k + kBlockK - 1u) / kBlockK;

  if (warp == 0) {
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool running = true;
      for (uint32_t tile = blockIdx.x; running && tile < tiles; tile += gridDim.x) {
        const uint32_t m0 = (tile % tiles_m) * kBlockM;
        const uint32_t n0 = (tile / tiles_m) * BN;
        for (uint32_t kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          ptx::mbarrier_arrive_expect_tx(&full[stage], L::kABytes + L::kBBytes);
          const int32_t x = static_cast<int32_t>(kt * kBlockK);
          ptx::tma_load_2d(shared_a + stage * L::kABytes, &map_a, &full[stage], x,
                           static_cast<int32_t>(m0));
          ptx::tma_load_2d(shared_b + stage * L::kBBytes, &map_b, &full[stage], x,
                           static_cast<int32_t>(n0));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort != 0u) {
        for (int spin = 0; spin < 256; ++spin) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      const uint32_t idesc = ptx::make_f16_idesc(input_type == kBf16, kBlockM, BN);
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      for (uint32_t tile = blockIdx.x; running && tile < tiles; tile += gridDim.x) {
        if (!ptx::mbarrier_wait(&acc_empty[acc_stage], acc_phase ^ 1u, abort)) break;
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * BN;
        for (uint32_t kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbarrier_wait(&full[stage], phase, abort)) {
            running = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint64_t a_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_a + stage * L::kABytes));
          const uint64_t b_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_b + stage * L::kBBytes));
#pragma unroll
          for (uint32_t kb = 0; kb < 4u; ++kb) {
            ptx::mma_f16(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc,
                         (kt | kb) != 0u);
          }
          ptx::tcgen05_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!running) break;
        ptx::tcgen05_commit(&acc_full[acc_stage]);
        if (++acc_stage == ACC_STAGES) {
          acc_stage = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    const uint32_t quarter = warp % 4u;
    uint32_t acc_stage = 0, acc_phase = 0;
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      const uint32_t m0 = (tile % tiles_m) * kBlockM;
      const uint32_t n0 = (tile / tiles_m) * BN;
      if (!ptx::mbarrier_wait(&acc_full[acc_stage], acc_phase, abort)) break;
      ptx::tcgen05_fence_after();
      const uint32_t row = m0 + quarter * 32u + lane;
      const uint32_t tmem_row = tmem_base + ((quarter * 32u) << 16) + acc_stage * BN;
#pragma unroll 1
      for (uint32_t chunk = 0; chunk < BN / 32u; ++chunk) {
        uint32_t values[32];
        ptx::tmem_load_32x32(tmem_row + chunk * 32u, values);
        ptx::tmem_load_wait();
        const uint32_t column = n0 + chunk * 32u;
        if (row < m && column < n) {
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
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbarrier_arrive(&acc_empty[acc_stage]);
      if (++acc_stage == ACC_STAGES) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tcgen05_fence_after();
    ptx::tmem_deallocate(tmem_base, kTmemColumns);
  }
  if (threadIdx.x == 0 && *abort != 0u) *status = 1u;
}

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
};

constexpr uint32_t kBlockN = 256, kStages = 4, kAccStages = 2;

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
        dense_gemm_kernel<kBlockN, kStages, kAccStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
        Layout<kBlockN, kStages, kAccStages>::kDynamicBytes));
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
    const int status = encode_operand(&plan->map_b, b, plan->n, plan->k, kBlockN);
    if (status != 0) return status;
    plan->cached_b = b;
  }
  const uint32_t tiles = ((plan->m + kBlockM - 1u) / kBlockM) * ((plan->n + kBlockN - 1u) / kBlockN);
  const uint32_t grid = tiles < static_cast<uint32_t>(plan->sm_count) ? tiles : plan->sm_count;
  dense_gemm_kernel<kBlockN, kStages, kAccStages>
      <<<grid, kThreads, Layout<kBlockN, kStages, kAccStages>::kDynamicBytes, cuda_stream>>>(
          plan->map_a, plan->map_b, c, plan->m, plan->n, plan->k, plan->input_type, plan->output_type,
          alpha, beta, plan->status);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" void mircuda_dense_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::dense_gemm::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
