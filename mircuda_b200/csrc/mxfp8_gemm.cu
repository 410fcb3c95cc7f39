// MXFP8 block-scaled GEMM for sm_100a: C[M,N] (bf16) = A[M,K] . B[N,K]^T with E4M3
// operands and one UE8M0 scale per 32 K-elements, fp32 accumulation in tensor memory.
//
// Replaces the reference's CUTLASS Sm120 instantiation (sys/native/mxfp8_sm120.cu) behind
// the same C entry points. Structure of one persistent CTA (192 threads, one CTA per SM):
//   warp 0   TMA producer: per 128-wide K step, A tile [128 x 128 B] and B tile
//            [BN x 128 B] by 2-D tensor maps with the 128-byte swizzle, plus the 512-byte
//            scale atoms of both operands by flat bulk copies (the global scale layout is
//            already the 32-lane x 16-byte block tcgen05.cp wants)
//   warp 1   MMA issuer: tcgen05.cp scales -> tensor memory, then four
//            tcgen05.mma.kind::mxf8f6f4.block_scale (K = 32 each) per stage; commits free
//            the shared-memory stage and, after the last K step, publish the accumulator
//   warps 2-5 epilogue: tcgen05.ld of their 32-lane quarter, fp32 -> bf16 (nearest even),
//            row-predicated 16-byte global stores
// Tiles are walked M-fastest so that the CTAs running together share B tiles and the whole
// of A stays in L2. Every mbarrier wait is bounded; a wait that runs out raises a flag that
// makes all roles leave, frees tensor memory and is reported through the plan status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <new>

#include "block_scaled_pair_gemm.cuh"
#include "layout.cuh"
#include "ptx.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace mxfp8_gemm {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kBlockK = 128;          // bytes == elements for E4M3
constexpr uint32_t kThreads = 192;
constexpr uint32_t kAtomBytes = 512;       // 128 rows x 4 scale columns
constexpr uint32_t kTmemColumns = 512;

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
struct Layout {
  static_assert(BN == 128 || BN == 192 || BN == 256, "supported tile widths");
  static constexpr uint32_t kABytes = kBlockM * kBlockK;
  static constexpr uint32_t kBBytes = BN * kBlockK;
  static constexpr uint32_t kSfbAtoms = BN == 128 ? 1 : 2;
  static constexpr uint32_t kAOffset = 0;
  static constexpr uint32_t kBOffset = STAGES * kABytes;
  static constexpr uint32_t kSfaOffset = kBOffset + STAGES * kBBytes;
  static constexpr uint32_t kSfbOffset = kSfaOffset + STAGES * kAtomBytes;
  static constexpr uint32_t kBarrierOffset = kSfbOffset + STAGES * kSfbAtoms * kAtomBytes;
  static constexpr uint32_t kBarriers = 2 * STAGES + 2 * ACC_STAGES;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  static constexpr uint32_t kBytes = kMiscOffset + 16;
  static constexpr uint32_t kDynamicBytes = kBytes + 1024;  // slack for 1024-byte alignment
  // Tensor memory: accumulators first, then 4 columns of A scales and 8 of B scales.
  static constexpr uint32_t kSfaColumn = ACC_STAGES * BN;
  static constexpr uint32_t kSfbColumn = kSfaColumn + 4;
  static_assert(kSfbColumn + 8 <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
__global__ void __launch_bounds__(kThreads, 1)
mxfp8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
       const uint8_t* __restrict__ scales_a, const uint8_t* __restrict__ scales_b,
       __nv_bfloat16* __restrict__ c, uint32_t m, uint32_t n, uint32_t k,
       uint32_t* __restrict__ status) {
  using L = Layout<BN, STAGES, ACC_STAGES>;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);

  uint8_t* shared_a = shared + L::kAOffset;
  uint8_t* shared_b = shared + L::kBOffset;
  uint8_t* shared_sfa = shared + L::kSfaOffset;
  uint8_t* shared_sfb = shared + L::kSfbOffset;
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
  const uint32_t k_tiles = k / kBlockK;
  const uint32_t atoms_n = (n + 127u) / 128u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool running = true;
      for (uint32_t tile = blockIdx.x; running && tile < tiles; tile += gridDim.x) {
        const uint32_t m0 = (tile % tiles_m) * kBlockM;
        const uint32_t n0 = (tile / tiles_m) * BN;
        const uint32_t first_atom = n0 / 128u;
        const uint32_t sfb_atoms = min(L::kSfbAtoms, atoms_n - first_atom);
        for (uint32_t kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          ptx::mbarrier_arrive_expect_tx(
              &full[stage], L::kABytes + L::kBBytes + kAtomBytes * (1u + sfb_atoms));
          ptx::tma_load_2d(shared_a + stage * L::kABytes, &map_a, &full[stage],
                           static_cast<int32_t>(kt * kBlockK), static_cast<int32_t>(m0));
          ptx::tma_load_2d(shared_b + stage * L::kBBytes, &map_b, &full[stage],
                           static_cast<int32_t>(kt * kBlockK), static_cast<int32_t>(n0));
          ptx::bulk_load(shared_sfa + stage * kAtomBytes,
                         scales_a + (static_cast<size_t>(m0 / 128u) * k_tiles + kt) * kAtomBytes,
                         kAtomBytes, &full[stage]);
          for (uint32_t atom = 0; atom < sfb_atoms; ++atom) {
            ptx::bulk_load(
                shared_sfb + (stage * L::kSfbAtoms + atom) * kAtomBytes,
                scales_b + (static_cast<size_t>(first_atom + atom) * k_tiles + kt) * kAtomBytes,
                kAtomBytes, &full[stage]);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort != 0u) {
        // Leave time for copies already issued to land before shared memory is released.
        for (int spin = 0; spin < 256; ++spin) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc =
          ptx::make_block_scaled_idesc(ptx::kFormatE4M3, ptx::kFormatE4M3, kBlockM, BN, true);
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      for (uint32_t tile = blockIdx.x; running && tile < tiles; tile += gridDim.x) {
        const uint32_t n0 = (tile / tiles_m) * BN;
        // A 192-wide tile may start in the middle of a 128-row scale atom: its first row is
        // then row 64 of the atom, i.e. two columns into the copied block.
        const uint32_t sfb_tmem = tmem_base + L::kSfbColumn + (n0 % 128u) / 32u;
        const uint32_t sfa_tmem = tmem_base + L::kSfaColumn;
        if (!ptx::mbarrier_wait(&acc_empty[acc_stage], acc_phase ^ 1u, abort)) break;
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * BN;
        for (uint32_t kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbarrier_wait(&full[stage], phase, abort)) {
            running = false;
            break;
          }
          ptx::tcgen05_fence_after();
          ptx::tcgen05_copy_scales(
              sfa_tmem,
              ptx::make_scale_descriptor(ptx::smem_address(shared_sfa + stage * kAtomBytes)));
#pragma unroll
          for (uint32_t atom = 0; atom < L::kSfbAtoms; ++atom) {
            ptx::tcgen05_copy_scales(
                tmem_base + L::kSfbColumn + 4u * atom,
                ptx::make_scale_descriptor(ptx::smem_address(
                    shared_sfb + (stage * L::kSfbAtoms + atom) * kAtomBytes)));
          }
          const uint64_t a_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_a + stage * L::kABytes));
          const uint64_t b_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_b + stage * L::kBBytes));
#pragma unroll
          for (uint32_t kb = 0; kb < 4u; ++kb) {
            // 32 bytes further along K inside the 128-byte swizzle span: +2 in 16-byte units.
            ptx::mma_mxf8f6f4_block_scale(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb,
                                          ptx::with_scale_ids(idesc, kb, kb), sfa_tmem, sfb_tmem,
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
    // ---------------------------------------------------------------------- epilogue
    const uint32_t quarter = warp % 4u;  // the 32 tensor-memory lanes this warp may read
    const bool vector_stores = (n % 8u) == 0u;
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
          __nv_bfloat16* destination = c + static_cast<size_t>(row) * n + column;
          if (vector_stores && column + 32u <= n) {
#pragma unroll
            for (uint32_t part = 0; part < 4u; ++part) {
              uint32_t packed[4];
#pragma unroll
              for (uint32_t pair = 0; pair < 4u; ++pair) {
                const __nv_bfloat162 two = __floats2bfloat162_rn(
                    __uint_as_float(values[part * 8u + pair * 2u]),
                    __uint_as_float(values[part * 8u + pair * 2u + 1u]));
                packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
              }
              reinterpret_cast<uint4*>(destination)[part] =
                  make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          } else {
#pragma unroll
            for (uint32_t item = 0; item < 32u; ++item) {
              if (column + item < n) {
                destination[item] = __float2bfloat16_rn(__uint_as_float(values[item]));
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

// ------------------------------------------------------------------------------- host

struct Plan {
  int m, n, k;
  int device;
  int sm_count;
  uint32_t block_n;
  cudaStream_t stream;
  uint32_t* status;        // pinned, device-visible; set by a kernel whose wait ran out
  const void* cached_a;
  const void* cached_b;
  CUtensorMap map_a, map_b;
  // CTA-pair kernel (used when M > 128): four tensor maps that depend on all four operands.
  bool pair;
  const void* cached_a_scales;
  const void* cached_b_scales;
  pair_gemm::Maps pair_maps;
};

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
int launch(Plan* plan, const void* a_scales, const void* b_scales, void* c) {
  using L = Layout<BN, STAGES, ACC_STAGES>;
  auto function = mxfp8_gemm_kernel<BN, STAGES, ACC_STAGES>;
  static thread_local int configured_device = -1;
  if (configured_device != plan->device) {
    const int status = static_cast<int>(cudaFuncSetAttribute(
        function, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
    if (status != 0) return status;
    configured_device = plan->device;
  }
  const uint32_t tiles = ((plan->m + kBlockM - 1u) / kBlockM) * ((plan->n + BN - 1u) / BN);
  const uint32_t grid = tiles < static_cast<uint32_t>(plan->sm_count)
                            ? tiles
                            : static_cast<uint32_t>(plan->sm_count);
  function<<<grid, kThreads, L::kDynamicBytes, plan->stream>>>(
      plan->map_a, plan->map_b, static_cast<const uint8_t*>(a_scales),
      static_cast<const uint8_t*>(b_scales), static_cast<__nv_bfloat16*>(c),
      static_cast<uint32_t>(plan->m), static_cast<uint32_t>(plan->n),
      static_cast<uint32_t>(plan->k), plan->status);
  return static_cast<int>(cudaPeekAtLastError());
}

// Tile width: fewest full waves of work, where a 128-wide tile pays for re-reading A from
// shared memory twice as often and a 256-wide tile cannot overlap its epilogue (one
// accumulator stage fits tensor memory next to the scale columns).
uint32_t choose_block_n(int m, int n, int k, int sm_count) {
  if (const char* forced = std::getenv("MIRCUDA_B200_GEMM_BN")) {
    const int value = std::atoi(forced);
    if (value == 128 || value == 192 || value == 256) return static_cast<uint32_t>(value);
  }
  const uint32_t candidates[3] = {256u, 192u, 128u};
  const double penalty[3] = {1.0 + 24.0 / (static_cast<double>(k) / 128.0 * 4.0 + 1.0), 1.0, 1.12};
  uint32_t best = 256u;
  double best_cost = 0.0;
  for (int index = 0; index < 3; ++index) {
    const uint32_t bn = candidates[index];
    const uint64_t tiles = static_cast<uint64_t>((m + 127) / 128) * ((n + bn - 1u) / bn);
    const uint64_t waves = (tiles + sm_count - 1) / sm_count;
    const double cost = static_cast<double>(waves) * bn * penalty[index];
    if (index == 0 || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

// Tile width for the CTA-pair kernel (256-row tiles on sm_count / 2 pairs): whole waves of
// work times a per-width cost. 256 columns leave room for one accumulator stage only, so the
// epilogue of a tile is exposed; 192 columns double-buffer the accumulator but move more
// shared-memory bytes per MMA cycle. (Widths that are not a multiple of 64 would make a tile
// start an odd number of columns into its scale block in tensor memory, which the MMA rejects
// as a misaligned address.)
uint32_t choose_pair_block_n(int m, int n, int k, int sm_count) {
  if (const char* forced = std::getenv("MIRCUDA_B200_GEMM_BN")) {
    const int value = std::atoi(forced);
    if (value == 128 || value == 192 || value == 256) return static_cast<uint32_t>(value);
  }
  const uint32_t candidates[3] = {256u, 192u, 128u};
  const double k_stages = static_cast<double>(k) / 128.0;
  // Measured on the prefill shapes: the 192-wide tile (two accumulator stages) beats the
  // 256-wide one (one stage, exposed epilogue) by 10-20 % at equal wave counts.
  const double penalty[3] = {1.12 + 2.0 / (k_stages + 1.0), 1.0, 1.30};
  const int pairs = sm_count / 2 > 0 ? sm_count / 2 : 1;
  uint32_t best = 256u;
  double best_cost = 0.0;
  for (int index = 0; index < 3; ++index) {
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

int execute_pair(Plan* plan, const void* a, const void* a_scales, const void* b,
                 const void* b_scales, void* c,
                 const pair_gemm::Gather& gather = pair_gemm::Gather{}) {
  using pair_gemm::Format;
  pair_gemm::Problem problem{static_cast<uint32_t>(plan->m), static_cast<uint32_t>(plan->n),
                             static_cast<uint32_t>(plan->k), plan->device, plan->sm_count,
                             plan->stream, plan->status};
  if (a != plan->cached_a || b != plan->cached_b || a_scales != plan->cached_a_scales ||
      b_scales != plan->cached_b_scales) {
    const int status = pair_gemm::encode_maps<Format::kMxFp8>(&plan->pair_maps, problem,
                                                              plan->block_n, a, a_scales, b, b_scales);
    if (status != 0) return status;
    plan->cached_a = a;
    plan->cached_b = b;
    plan->cached_a_scales = a_scales;
    plan->cached_b_scales = b_scales;
  }
  switch (plan->block_n) {
    case 128u:
      return pair_gemm::launch<Format::kMxFp8, 128u, 8u, 2u>(problem, plan->pair_maps, c, 1.0f,
                                                             gather);
    case 192u:
      return pair_gemm::launch<Format::kMxFp8, 192u, 7u, 2u>(problem, plan->pair_maps, c, 1.0f,
                                                             gather);
    default:
      return pair_gemm::launch<Format::kMxFp8, 256u, 6u, 1u>(problem, plan->pair_maps, c, 1.0f,
                                                             gather);
  }
}

}  // namespace mxfp8_gemm
}  // namespace mircuda_b200

extern "C" int mircuda_mxfp8_tc_create(int m, int n, int k, void* stream, void** output) {
  using namespace mircuda_b200::mxfp8_gemm;
  if (m <= 0 || n <= 0 || k <= 0 || k % 128 != 0 || stream == nullptr || output == nullptr) {
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
  const char* mode = std::getenv("MIRCUDA_B200_GEMM_PAIR");   // "0" forces the unpaired kernel
  plan->pair = m > 128 && plan->sm_count >= 2 && !(mode != nullptr && mode[0] == '0');
  plan->block_n = plan->pair ? choose_pair_block_n(m, n, k, plan->sm_count)
                             : choose_block_n(m, n, k, plan->sm_count);
  *output = plan;
  return 0;
}

extern "C" size_t mircuda_mxfp8_tc_workspace_bytes(const void* raw) {
  // The kernel needs no device workspace: partial sums never leave tensor memory.
  (void)raw;
  return 0;
}

extern "C" int mircuda_mxfp8_tc_execute(void* raw, void* stream, const void* a,
                                        const void* a_scales, const void* b,
                                        const void* b_scales, void* c) {
  using namespace mircuda_b200;
  using namespace mircuda_b200::mxfp8_gemm;
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
  if (plan->pair) return execute_pair(plan, a, a_scales, b, b_scales, c);
  if (a != plan->cached_a) {
    const int status = encode_k_major_map(&plan->map_a, a, plan->m, plan->k, 1u, kBlockM);
    if (status != 0) return status;
    plan->cached_a = a;
  }
  if (b != plan->cached_b) {
    const int status = encode_k_major_map(&plan->map_b, b, plan->n, plan->k, 1u, plan->block_n);
    if (status != 0) return status;
    plan->cached_b = b;
  }
  switch (plan->block_n) {
    case 128u: return launch<128u, 6u, 2u>(plan, a_scales, b_scales, c);
    case 192u: return launch<192u, 5u, 2u>(plan, a_scales, b_scales, c);
    default: return launch<256u, 4u, 1u>(plan, a_scales, b_scales, c);
  }
}

extern "C" int mircuda_b200_mxfp8_tc_execute_gather(void* raw, void* stream, const void* a,
                                                    const void* a_scales, const void* b,
                                                    const void* b_scales, void* const* outputs,
                                                    int output_count, int row_stride,
                                                    int column_offset, void* multicast_output) {
  using namespace mircuda_b200;
  using namespace mircuda_b200::mxfp8_gemm;
  if (raw == nullptr || stream == nullptr || a == nullptr || a_scales == nullptr ||
      b == nullptr || b_scales == nullptr || outputs == nullptr || output_count <= 0 ||
      output_count > 8 || row_stride <= 0 || column_offset < 0) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  if (static_cast<cudaStream_t>(stream) != plan->stream) return -1;
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  // The fused path lives in the CTA-pair kernel and stores 16-byte vectors.
  if (!plan->pair || plan->n % 8 != 0 || row_stride % 8 != 0 || column_offset % 8 != 0 ||
      column_offset + plan->n > row_stride) {
    return -1;
  }
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
        reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(b_scales)) & 15u) != 0u) {
    return -1;
  }
  pair_gemm::Gather gather{};
  for (int index = 0; index < output_count; ++index) {
    if (outputs[index] == nullptr || (reinterpret_cast<uintptr_t>(outputs[index]) & 15u) != 0u) return -1;
    gather.outputs[index] = static_cast<__nv_bfloat16*>(outputs[index]);
  }
  gather.multicast = static_cast<__nv_bfloat16*>(multicast_output);
  gather.count = static_cast<uint32_t>(output_count);
  gather.row_stride = static_cast<uint32_t>(row_stride);
  gather.column_offset = static_cast<uint32_t>(column_offset);
  return execute_pair(plan, a, a_scales, b, b_scales, outputs[0], gather);
}

namespace mircuda_b200 {
namespace mxfp8_gemm {

// One warp waits, with a 2 ms budget instead of the kernels' half second, on a barrier that
// nothing ever arrives at, and leaves the way the GEMM roles leave when a wait runs out: the
// wait raises the CTA's abort flag and returns false, and thread 0 reports it through the
// plan's status word. The kernel always returns by itself.
__global__ void __launch_bounds__(32) wait_probe_kernel(uint32_t* __restrict__ status) {
  __shared__ uint64_t barrier;
  __shared__ uint32_t abort_flag;
  volatile uint32_t* abort = &abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbarrier_init(&barrier, 1);
    *abort = 0u;
    ptx::fence_barrier_init();
  }
  __syncwarp();
  ptx::mbarrier_wait<2ull * 1000ull * 1000ull>(&barrier, 0u, abort);
  __syncwarp();
  if (threadIdx.x == 0 && *abort != 0u) *status = 1u;
}

}  // namespace mxfp8_gemm
}  // namespace mircuda_b200

extern "C" int mircuda_b200_mxfp8_tc_wait_probe(void* raw, void* stream) {
  using namespace mircuda_b200::mxfp8_gemm;
  if (raw == nullptr || stream == nullptr) return -1;
  auto* plan = static_cast<Plan*>(raw);
  if (static_cast<cudaStream_t>(stream) != plan->stream) return -1;
  wait_probe_kernel<<<1, 32, 0, plan->stream>>>(plan->status);
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" void mircuda_mxfp8_tc_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::mxfp8_gemm::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
