// The tile kernel of dense_tile.cuh on CTA pairs (tcgen05.mma.cta_group::2), used by the dense
// f16 / bf16 GEMM and the scaled FP8 GEMM above 128 rows of A: a cluster of two CTAs owns a tile
// of 256 rows of A x BN rows of B; each CTA loads its own 128 rows of A and its half of the B
// rows, the leader's MMA warp issues the instructions for both SMs, every CTA drains its own
// 128 accumulator rows. A single CTA with a 128 x 256 tile is bound by its shared-memory port:
// per stage its MMAs read 48 KB that TMA first wrote, 96 KB through a 128-byte-per-clock port
// against 512 clocks of MMA time; a pair moves two thirds of that per flop.
//
// Roles as in dense_tile.cuh (warp 0 TMA, warp 1 MMA in the leader CTA only, warps 2-5
// epilogue). The barriers the MMA issuer waits on live in the leader CTA: both CTAs' loads are
// counted there, both CTAs' epilogue warps arrive there; the issuer releases stages and
// announces accumulators in both CTAs with multicast commits. Every wait is bounded; a wait that
// gives up raises the CTA's abort flag, every role leaves its loop, tensor memory is freed and
// *status is set.
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "launch_overlap.hpp"
#include "ptx.cuh"
#include "ptx_pair.cuh"

namespace mircuda_b200 {
namespace dense_pair {

constexpr uint32_t kBlockM = 128;          // rows of A per CTA; a pair tile has 256
constexpr uint32_t kBlockKBytes = 128;
constexpr uint32_t kThreads = 192;
constexpr uint32_t kTmemColumns = 512;

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
struct Layout {
  static constexpr uint32_t kABytes = kBlockM * kBlockKBytes;
  static constexpr uint32_t kBBytes = (BN / 2u) * kBlockKBytes;      // this CTA's half of the B rows
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kBOffset = STAGES * kABytes;
  static constexpr uint32_t kBarrierOffset = kBOffset + STAGES * kBBytes;
  static constexpr uint32_t kBarriers = 2 * STAGES + 2 * ACC_STAGES;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  static constexpr uint32_t kDynamicBytes = kMiscOffset + 16 + 1024;
  static_assert(ACC_STAGES * BN <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES, typename Epilogue>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
dense_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  uint32_t m, uint32_t n, uint32_t k, uint32_t idesc, const Epilogue epilogue,
                  uint32_t* __restrict__ status) {
  using L = Layout<BN, STAGES, ACC_STAGES>;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_a = shared;
  uint8_t* shared_b = shared + L::kBOffset;
  uint64_t* full = reinterpret_cast<uint64_t*>(shared + L::kBarrierOffset);   // leader's
  uint64_t* empty = full + STAGES;                                             // each CTA
  uint64_t* acc_full = empty + STAGES;                                         // each CTA
  uint64_t* acc_empty = acc_full + ACC_STAGES;                                 // leader's
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(shared + L::kMiscOffset);
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const uint32_t warp = threadIdx.x / 32u;
  const uint32_t lane = threadIdx.x % 32u;
  const uint32_t rank = ptx::cluster_cta_rank();   // 0 = leader
  const bool leader = rank == 0u;

  if (threadIdx.x == 0) {
    for (uint32_t stage = 0; stage < STAGES; ++stage) {
      ptx::mbarrier_init(&full[stage], 2);          // one arrive.expect_tx per CTA
      ptx::mbarrier_init(&empty[stage], 1);         // one commit arrival
    }
    for (uint32_t stage = 0; stage < ACC_STAGES; ++stage) {
      ptx::mbarrier_init(&acc_full[stage], 1);
      ptx::mbarrier_init(&acc_empty[stage], 8);     // four epilogue warps in each CTA
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&map_a);
    ptx::prefetch_tensor_map(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_allocate_pair(tmem_slot, kTmemColumns);
    ptx::tmem_relinquish_pair();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Nothing above touched global memory; the rest runs after the kernel before this one.
  ptx::dependency_launch_next();
  ptx::dependency_wait();

  const uint32_t tiles_m = (m + 2u * kBlockM - 1u) / (2u * kBlockM);
  const uint32_t tiles_n = (n + BN - 1u) / BN;
  const uint32_t tiles = tiles_m * tiles_n;
  constexpr uint32_t kBlockK = kBlockKBytes / Epilogue::kElementBytes;
  const uint32_t k_tiles = (k + kBlockK - 1u) / kBlockK;
  const uint32_t pair = blockIdx.x / 2u;
  const uint32_t pairs = gridDim.x / 2u;

  if (warp == 0) {
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool running = true;
      for (uint32_t tile = pair; running && tile < tiles; tile += pairs) {
        const uint32_t m0 = (tile % tiles_m) * 2u * kBlockM + rank * kBlockM;
        const uint32_t n0 = (tile / tiles_m) * BN + rank * (BN / 2u);
        for (uint32_t kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          // Every byte this CTA loads is counted on the leader's barrier of the stage.
          const uint32_t barrier = ptx::map_to_cta(ptx::smem_address(&full[stage]), 0u);
          ptx::mbarrier_arrive_expect_tx_cluster(barrier, L::kStageBytes);
          const int32_t x = static_cast<int32_t>(kt * kBlockK);
          ptx::tma_load_2d_pair(shared_a + stage * L::kABytes, &map_a, barrier, x, static_cast<int32_t>(m0));
          ptx::tma_load_2d_pair(shared_b + stage * L::kBBytes, &map_b, barrier, x, static_cast<int32_t>(n0));
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
    if (leader && ptx::elect_one()) {
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      for (uint32_t tile = pair; running && tile < tiles; tile += pairs) {
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
            if constexpr (Epilogue::kElementBytes == 1u) {
              ptx::mma_f8f6f4_pair(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc,
                                   (kt | kb) != 0u);
            } else {
              ptx::mma_f16_pair(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc, (kt | kb) != 0u);
            }
          }
          ptx::tcgen05_commit_pair(&empty[stage], 3u);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!running) break;
        ptx::tcgen05_commit_pair(&acc_full[acc_stage], 3u);
        if (++acc_stage == ACC_STAGES) {
          acc_stage = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    const uint32_t quarter = warp % 4u;
    uint32_t acc_stage = 0, acc_phase = 0;
    for (uint32_t tile = pair; tile < tiles; tile += pairs) {
      const uint32_t m0 = (tile % tiles_m) * 2u * kBlockM + rank * kBlockM;
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
        if (row < m && column < n) epilogue.store(row, column, values, n);
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        ptx::mbarrier_arrive_cluster(ptx::map_to_cta(ptx::smem_address(&acc_empty[acc_stage]), 0u));
      }
      if (++acc_stage == ACC_STAGES) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // Neither CTA may free tensor memory or exit while the other can still signal its barriers
  // or while the leader's MMAs still read its shared memory.
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    __syncwarp();
    ptx::tcgen05_fence_after();
    ptx::tmem_deallocate_pair(tmem_base, kTmemColumns);
  }
  if (threadIdx.x == 0 && *abort != 0u) *status = 1u;
}

// Sets the kernel's shared-memory attribute and asks how many pairs the device holds at once
// (the kernel is persistent: every pair must be resident, and not every SM can be paired).
template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES, typename Epilogue>
int prepare(int sm_count, int* resident_pairs) {
  using L = Layout<BN, STAGES, ACC_STAGES>;
  auto function = dense_pair_kernel<BN, STAGES, ACC_STAGES, Epilogue>;
  int status = static_cast<int>(cudaFuncSetAttribute(function, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     L::kDynamicBytes));
  if (status != 0) return status;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned int>(sm_count) & ~1u, 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = L::kDynamicBytes;
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 2;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  status = static_cast<int>(cudaOccupancyMaxActiveClusters(&clusters, function, &config));
  if (status != 0) return status;
  if (clusters < 1) return static_cast<int>(cudaErrorLaunchOutOfResources);
  *resident_pairs = clusters;
  return 0;
}

// `map_b` must have been encoded with boxes of BN / 2 rows.
template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES, typename Epilogue>
int launch(cudaStream_t stream, int resident_pairs, const CUtensorMap& map_a, const CUtensorMap& map_b, uint32_t m,
           uint32_t n, uint32_t k, uint32_t idesc, const Epilogue& epilogue, uint32_t* status) {
  using L = Layout<BN, STAGES, ACC_STAGES>;
  const uint32_t tiles = ((m + 2u * kBlockM - 1u) / (2u * kBlockM)) * ((n + BN - 1u) / BN);
  const uint32_t pairs = tiles < static_cast<uint32_t>(resident_pairs) ? tiles : resident_pairs;
  return launch_after_dependency(dense_pair_kernel<BN, STAGES, ACC_STAGES, Epilogue>, dim3(2u * pairs),
                                 dim3(kThreads), L::kDynamicBytes, stream, map_a, map_b, m, n, k, idesc, epilogue,
                                 status);
}

}  // namespace dense_pair
}  // namespace mircuda_b200
