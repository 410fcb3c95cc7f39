// Persistent tcgen05 tile kernel shared by the dense f16 / bf16 GEMM and the scaled FP8 GEMM:
// C[M,N] = epilogue(A[M,K] . B[N,K]^T), operands K-major, fp32 accumulation in tensor memory.
// One 192-thread CTA per SM: warp 0 issues TMA loads of 128-byte-swizzled tiles (A 128 rows,
// B BN rows, 128 bytes of K per stage), warp 1 issues four tcgen05.mma per stage (32 bytes of K
// each; kind::f16 for two-byte elements, kind::f8f6f4 for one-byte e4m3), warps 2-5 read the
// accumulator back 32 columns at a time and hand each lane's row segment to Epilogue::store.
// Tiles are walked M-fastest so that CTAs running together share B tiles. Every mbarrier wait
// is bounded; a wait that gives up sets *status and the kernel returns after freeing its
// tensor memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "ptx.cuh"

namespace mircuda_b200 {
namespace dense_tile {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kBlockKBytes = 128;     // 64 two-byte elements per stage row
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

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES, typename Epilogue>
__global__ void __launch_bounds__(kThreads, 1)
dense_tile_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  uint32_t m, uint32_t n, uint32_t k, uint32_t idesc, const Epilogue epilogue,
                  uint32_t* __restrict__ status) {
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
  constexpr uint32_t kBlockK = kBlockKBytes / Epilogue::kElementBytes;
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
            if constexpr (Epilogue::kElementBytes == 1u) {
              ptx::mma_f8f6f4(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc,
                              (kt | kb) != 0u);
            } else {
              ptx::mma_f16(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc,
                           (kt | kb) != 0u);
            }
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
        if (row < m && column < n) epilogue.store(row, column, values, n);
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

}  // namespace dense_tile
}  // namespace mircuda_b200
