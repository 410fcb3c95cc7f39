// NVFP4 block-scaled GEMM: C[M,N] (bf16) = alpha * A[M,K] . B[N,K]^T with E2M1 operands (two
// codes per byte, even k in the low nibble) and one UE4M3 scale per 16 K-elements in the
// 128x4-swizzled layout; fp32 accumulation. Replaces the reference's CUTLASS Sm120
// instantiation (sys/native/fp4_sm120.cu:110-170) behind the same C entry points, on the
// CTA-pair tcgen05 kernel (kind::mxf4nvf4, block16) of block_scaled_pair_gemm.cuh.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <new>

#include "block_scaled_pair_gemm.cuh"

namespace mircuda_b200 {
namespace fp4_gemm {

struct Plan {
  int m, n, k;
  int device, sm_count;
  uint32_t block_n;
  cudaStream_t stream;
  uint32_t* status;
  const void* cached[4];
  pair_gemm::Maps maps;
};

uint32_t choose_block_n(int m, int n, int k, int sm_count) {
  if (const char* forced = std::getenv("MIRCUDA_B200_FP4_GEMM_BN")) {
    const int value = std::atoi(forced);
    if (value == 128 || value == 192 || value == 256) return static_cast<uint32_t>(value);
  }
  if (n <= 128) return 128u;
  const uint32_t candidates[2] = {256u, 192u};
  const double k_stages = static_cast<double>(k) / 256.0;
  const double penalty[2] = {1.12 + 2.0 / (k_stages + 1.0), 1.0};
  const int pairs = sm_count / 2 > 0 ? sm_count / 2 : 1;
  uint32_t best = 256u;
  double best_cost = 0.0;
  for (int index = 0; index < 2; ++index) {
    const uint32_t bn = candidates[index];
    const uint64_t tiles = static_cast<uint64_t>((m + 255) / 256) * ((n + bn - 1u) / bn);
    const uint64_t waves = (tiles + pairs - 1) / pairs;
    const double cost = static_cast<double>(waves) * bn * penalty[index];
    if (index == 0 || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

}  // namespace fp4_gemm
}  // namespace mircuda_b200

extern "C" int mircuda_fp4_create(int m, int n, int k, void* stream, void** output) {
  using namespace mircuda_b200::fp4_gemm;
  if (m <= 0 || n <= 0 || k <= 0 || k % 64 != 0 || stream == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->m = m;
  plan->n = n;
  plan->k = k;
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
  if (status != 0) {
    delete plan;
    return status;
  }
  *plan->status = 0u;
  plan->block_n = choose_block_n(m, n, k, plan->sm_count);
  *output = plan;
  return 0;
}

extern "C" size_t mircuda_fp4_workspace_bytes(const void* raw) {
  (void)raw;
  return 0;  // partial sums never leave tensor memory
}

extern "C" int mircuda_fp4_execute(void* raw, void* stream, const void* a, const void* a_scales,
                                   const void* b, const void* b_scales, void* c, float alpha) {
  using namespace mircuda_b200;
  using namespace mircuda_b200::fp4_gemm;
  using pair_gemm::Format;
  if (raw == nullptr || stream == nullptr || a == nullptr || a_scales == nullptr ||
      b == nullptr || b_scales == nullptr || c == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  if (static_cast<cudaStream_t>(stream) != plan->stream) return -1;
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
        reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(b_scales)) & 15u) != 0u) {
    return -1;
  }
  // With n a multiple of 8 the epilogue writes 16-byte vectors: the output must allow them.
  if (plan->n % 8 == 0 && (reinterpret_cast<uintptr_t>(c) & 15u) != 0u) return -1;
  pair_gemm::Problem problem{static_cast<uint32_t>(plan->m), static_cast<uint32_t>(plan->n),
                             static_cast<uint32_t>(plan->k), plan->device, plan->sm_count,
                             plan->stream, plan->status};
  const void* operands[4] = {a, a_scales, b, b_scales};
  bool changed = false;
  for (int index = 0; index < 4; ++index) changed |= operands[index] != plan->cached[index];
  if (changed) {
    const int status = pair_gemm::encode_maps<Format::kNvFp4>(&plan->maps, problem, plan->block_n, a,
                                                              a_scales, b, b_scales);
    if (status != 0) return status;
    for (int index = 0; index < 4; ++index) plan->cached[index] = operands[index];
  }
  switch (plan->block_n) {
    case 128u:
      return pair_gemm::launch<Format::kNvFp4, 128u, 7u, 2u>(problem, plan->maps, c, alpha);
    case 192u:
      return pair_gemm::launch<Format::kNvFp4, 192u, 6u, 2u>(problem, plan->maps, c, alpha);
    default:
      return pair_gemm::launch<Format::kNvFp4, 256u, 5u, 1u>(problem, plan->maps, c, alpha);
  }
}

extern "C" void mircuda_fp4_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::fp4_gemm::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
