// int4-g128 W4A16 GEMM for prefill on CTA pairs (M > 128): the fused GEMM of w4a16_tile.cu with
// tcgen05.mma.cta_group::2. A pair of CTAs (a cluster of two) owns a tile of 256 tokens x 256
// weight rows; each CTA loads its own 128 token rows and expands only its own 128 weight rows,
// and the tensor cores of both SMs read both halves. Against single-CTA tiles this halves the
// expansion work per tile (two CTAs on the two token halves of one weight tile both expanded all
// of it) and the shared-memory traffic per flop, which is what bounds a 128 x 256 f16 tile:
// per 64-element stage its MMAs read 48 KB that TMA and the converters first wrote, 112 KB in
// all through a 128-byte-per-clock port, against 512 clocks of MMA time.
//
// Per CTA, 448 threads: warp 0 issues the TMA loads (activation tile every stage, packed weight
// rows of two stages every other stage), warp 1 of the leader CTA issues the MMAs for the pair,
// warps 2-5 drain this CTA's half of the accumulator, warps 6-13 (two groups that take the
// stages in turn, one weight row per thread) expand packed rows into the K-major 128-byte-
// swizzled B half-tile. Barriers the MMA issuer waits on live in the leader CTA (the peer's
// loads and converters signal them across the cluster); the issuer releases stages in both
// CTAs with multicast commits. Every wait is bounded; a wait that gives up raises the CTA's
// abort flag, every role leaves its loop, tensor memory is freed and *status is set.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "launch_overlap.hpp"
#include "ptx.cuh"
#include "ptx_pair.cuh"
#include "tensor_map.hpp"
#include "w4a16_expand.cuh"
#include "w4a16_tile.hpp"

namespace mircuda_b200 {
namespace w4a16_pair {

using namespace w4a16_expand;

constexpr uint32_t kBlockM = 128;          // token rows per CTA; a pair tile has 256
constexpr uint32_t kBlockN = 256;          // weight rows per pair tile; a CTA expands 128
constexpr uint32_t kHalfN = kBlockN / 2u;
constexpr uint32_t kBlockK = 64;
constexpr uint32_t kGroupK = 128;
constexpr uint32_t kConverterThreads = 256;
constexpr uint32_t kConverterGroups = 2;
constexpr uint32_t kGroupThreads = kConverterThreads / kConverterGroups;   // 128 = rows a CTA expands
constexpr uint32_t kThreads = 6u * 32u + kConverterThreads;
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kChapterGroups = 16;
constexpr uint32_t kStages = 6;            // activation tiles
constexpr uint32_t kBStages = 4;           // expanded weight half-tiles
constexpr uint32_t kPackedStages = 2;      // packed tiles, each the rows' bytes of two stages
constexpr uint32_t kAccStages = 2;

struct Layout {
  static constexpr uint32_t kABytes = kBlockM * 128u;              // 16 KB
  static constexpr uint32_t kBBytes = kHalfN * 128u;               // 16 KB
  static constexpr uint32_t kPackedBytes = kHalfN * 64u;           // 8 KB
  static constexpr uint32_t kBOffset = kStages * kABytes;
  static constexpr uint32_t kPackedOffset = kBOffset + kBStages * kBBytes;
  static constexpr uint32_t kScaleOffset = kPackedOffset + kPackedStages * kPackedBytes;   // [group][scale group][row]
  static constexpr uint32_t kBarrierOffset = kScaleOffset + kConverterGroups * kChapterGroups * kHalfN * 2u;
  static constexpr uint32_t kBarriers = 2 * kStages + 2 * kBStages + 2 * kPackedStages + 2 * kAccStages;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  static constexpr uint32_t kDynamicBytes = kMiscOffset + 16 + 1024;
  static_assert(kAccStages * kBlockN <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
w4a16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                  const __half* __restrict__ scales, __half* __restrict__ c, float* __restrict__ partial,
                  uint32_t m, uint32_t n, uint32_t k, uint32_t splits, uint32_t idesc,
                  uint32_t* __restrict__ status) {
  using L = Layout;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_a = shared;
  uint8_t* shared_b = shared + L::kBOffset;
  uint8_t* shared_packed = shared + L::kPackedOffset;
  uint64_t* loaded = reinterpret_cast<uint64_t*>(shared + L::kBarrierOffset);   // leader's: both CTAs' TMA -> MMA
  uint64_t* empty = loaded + kStages;                                            // MMA -> TMA (each CTA)
  uint64_t* converted = empty + kStages;                                         // leader's: converters -> MMA
  uint64_t* b_empty = converted + kBStages;                                      // MMA -> converters (each CTA)
  uint64_t* packed_full = b_empty + kBStages;                                    // TMA -> converters (local)
  uint64_t* packed_empty = packed_full + kPackedStages;                          // converters -> TMA (local)
  uint64_t* acc_full = packed_empty + kPackedStages;                             // MMA -> epilogue (each CTA)
  uint64_t* acc_empty = acc_full + kAccStages;                                   // leader's: both epilogues -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(shared + L::kMiscOffset);
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const uint32_t warp = threadIdx.x / 32u;
  const uint32_t lane = threadIdx.x % 32u;
  const uint32_t rank = ptx::cluster_cta_rank();   // 0 = leader
  const bool leader = rank == 0u;

  if (threadIdx.x == 0) {
    for (uint32_t stage = 0; stage < kStages; ++stage) {
      ptx::mbarrier_init(&loaded[stage], 2);                            // one arrive.expect_tx per CTA
      ptx::mbarrier_init(&empty[stage], 1);                             // one commit arrival
    }
    for (uint32_t stage = 0; stage < kBStages; ++stage) {
      ptx::mbarrier_init(&converted[stage], 2u * kGroupThreads / 32u);  // a group's warps in each CTA
      ptx::mbarrier_init(&b_empty[stage], 1);
    }
    for (uint32_t stage = 0; stage < kPackedStages; ++stage) {
      ptx::mbarrier_init(&packed_full[stage], 1);
      ptx::mbarrier_init(&packed_empty[stage], kConverterThreads / 32u);
    }
    for (uint32_t stage = 0; stage < kAccStages; ++stage) {
      ptx::mbarrier_init(&acc_full[stage], 1);
      ptx::mbarrier_init(&acc_empty[stage], 8);                         // four epilogue warps in each CTA
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&map_a);
    ptx::prefetch_tensor_map(&map_w);
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
  const uint32_t tiles_n = (n + kBlockN - 1u) / kBlockN;
  const uint32_t tiles = tiles_m * tiles_n;
  const uint32_t units = tiles * splits;             // unit = tile + split * tiles
  const uint32_t k_tiles = k / kBlockK / splits;     // per unit (an even number: whole scale groups)
  const uint32_t pair = blockIdx.x / 2u;
  const uint32_t pairs = gridDim.x / 2u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0, packed_stage = 0, packed_phase = 0;
      bool running = true;
      for (uint32_t unit = pair; running && unit < units; unit += pairs) {
        const uint32_t tile = unit % tiles;
        const uint32_t first_kt = (unit / tiles) * k_tiles;
        const uint32_t m0 = (tile % tiles_m) * 2u * kBlockM + rank * kBlockM;
        const uint32_t n0 = (tile / tiles_m) * kBlockN + rank * kHalfN;
        for (uint32_t kt = first_kt; kt < first_kt + k_tiles; ++kt) {
          if ((kt - first_kt) % 2u == 0u) {
            // This CTA's packed weight rows of the next two stages.
            if (!ptx::mbarrier_wait<ptx::kWaitBudgetNs, 64u>(&packed_empty[packed_stage], packed_phase ^ 1u, abort)) {
              running = false;
              break;
            }
            ptx::mbarrier_arrive_expect_tx(&packed_full[packed_stage], L::kPackedBytes);
            ptx::tma_load_2d(shared_packed + packed_stage * L::kPackedBytes, &map_w, &packed_full[packed_stage],
                             static_cast<int32_t>(kt * (kBlockK / 2u)), static_cast<int32_t>(n0));
            if (++packed_stage == kPackedStages) {
              packed_stage = 0;
              packed_phase ^= 1u;
            }
          }
          if (!ptx::mbarrier_wait<ptx::kWaitBudgetNs, 64u>(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          // The bytes this CTA loads are counted on the leader's barrier of the stage.
          const uint32_t barrier = ptx::map_to_cta(ptx::smem_address(&loaded[stage]), 0u);
          ptx::mbarrier_arrive_expect_tx_cluster(barrier, L::kABytes);
          ptx::tma_load_2d_pair(shared_a + stage * L::kABytes, &map_a, barrier,
                                static_cast<int32_t>(kt * kBlockK), static_cast<int32_t>(m0));
          if (++stage == kStages) {
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
    // ------------------------------------------------------- MMA issuer (leader CTA only)
    if (leader && ptx::elect_one()) {
      uint32_t stage = 0, phase = 0, b_stage = 0, b_phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      for (uint32_t unit = pair; running && unit < units; unit += pairs) {
        if (!ptx::mbarrier_wait<ptx::kWaitBudgetNs, 64u>(&acc_empty[acc_stage], acc_phase ^ 1u, abort)) break;
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * kBlockN;
        for (uint32_t kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbarrier_wait<ptx::kWaitBudgetNs, 32u>(&loaded[stage], phase, abort) ||
              !ptx::mbarrier_wait<ptx::kWaitBudgetNs, 32u>(&converted[b_stage], b_phase, abort)) {
            running = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint64_t a_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_a + stage * L::kABytes));
          const uint64_t b_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_b + b_stage * L::kBBytes));
#pragma unroll
          for (uint32_t kb = 0; kb < 4u; ++kb) {
            ptx::mma_f16_pair(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc, (kt | kb) != 0u);
          }
          // Both CTAs' activation tiles and expanded half-tiles of the stage are free again.
          ptx::tcgen05_commit_pair(&empty[stage], 3u);
          ptx::tcgen05_commit_pair(&b_empty[b_stage], 3u);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++b_stage == kBStages) {
            b_stage = 0;
            b_phase ^= 1u;
          }
        }
        if (!running) break;
        ptx::tcgen05_commit_pair(&acc_full[acc_stage], 3u);
        if (++acc_stage == kAccStages) {
          acc_stage = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp < 6u) {
    // ------------------------------------------------------------------ epilogue
    const uint32_t quarter = warp % 4u;
    uint32_t acc_stage = 0, acc_phase = 0;
    for (uint32_t unit = pair; unit < units; unit += pairs) {
      const uint32_t tile = unit % tiles;
      const uint32_t m0 = (tile % tiles_m) * 2u * kBlockM + rank * kBlockM;
      const uint32_t n0 = (tile / tiles_m) * kBlockN;
      float* partial_rows = partial + static_cast<size_t>(unit / tiles) * m * n;
      // The epilogue warps wait for a whole tile's main loop beside the converters: sleep between polls.
      if (!ptx::mbarrier_wait<ptx::kWaitBudgetNs, 256u>(&acc_full[acc_stage], acc_phase, abort)) break;
      ptx::tcgen05_fence_after();
      const uint32_t row = m0 + quarter * 32u + lane;
      const uint32_t tmem_row = tmem_base + ((quarter * 32u) << 16) + acc_stage * kBlockN;
#pragma unroll 1
      for (uint32_t chunk = 0; chunk < kBlockN / 32u; ++chunk) {
        uint32_t values[32];
        ptx::tmem_load_32x32(tmem_row + chunk * 32u, values);
        ptx::tmem_load_wait();
        const uint32_t column = n0 + chunk * 32u;
        if (row < m && column < n && splits > 1u) {
          // fp32 partial tile of this K range; n % 8 == 0 makes the pieces 16-byte aligned
          float* destination = partial_rows + static_cast<size_t>(row) * n + column;
#pragma unroll
          for (uint32_t part = 0; part < 8u; ++part) {
            if (column + part * 4u < n) {
              reinterpret_cast<uint4*>(destination)[part] = make_uint4(values[part * 4u], values[part * 4u + 1u],
                                                                      values[part * 4u + 2u], values[part * 4u + 3u]);
            }
          }
        } else if (row < m && column < n) {
          __half* destination = c + static_cast<size_t>(row) * n + column;
          if (column + 32u <= n) {       // n % 8 == 0 and a 16-byte aligned base: 16-byte stores
#pragma unroll
            for (uint32_t part = 0; part < 4u; ++part) {
              uint32_t packed[4];
#pragma unroll
              for (uint32_t pair_index = 0; pair_index < 4u; ++pair_index) {
                const __half2 two = __floats2half2_rn(__uint_as_float(values[part * 8u + pair_index * 2u]),
                                                      __uint_as_float(values[part * 8u + pair_index * 2u + 1u]));
                packed[pair_index] = *reinterpret_cast<const uint32_t*>(&two);
              }
              reinterpret_cast<uint4*>(destination)[part] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          } else {
#pragma unroll
            for (uint32_t item = 0; item < 32u; ++item) {
              if (column + item < n) destination[item] = __float2half_rn(__uint_as_float(values[item]));
            }
          }
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        ptx::mbarrier_arrive_cluster(ptx::map_to_cta(ptx::smem_address(&acc_empty[acc_stage]), 0u));
      }
      if (++acc_stage == kAccStages) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ converters
    // Two groups of four warps take the stages in turn (group g the stages with kt % 2 == g, a
    // thread one of this CTA's 128 weight rows), so that two stages are being expanded at any
    // time.
    const uint32_t group = (threadIdx.x - 6u * 32u) / kGroupThreads;
    const uint32_t thread = (threadIdx.x - 6u * 32u) % kGroupThreads;
    const uint32_t groups_k = k / kGroupK;
    const uint32_t unit_groups = k_tiles / 2u;
    // The row's scales of the next kChapterGroups scale groups live in shared memory, one table
    // per converter group, [scale group][row]; a thread writes and reads only its own column.
    // (Global loads are kept out of the stage loop: the proxy fence at the end of a stage waits
    // for every load the thread still has in flight.)
    const uint32_t table = ptx::smem_address(shared + L::kScaleOffset) + group * (kChapterGroups * kHalfN * 2u) +
                           thread * 2u;
    // Ring positions advance with every stage, also the other group's.
    uint32_t packed_stage = 0, packed_phase = 0, b_stage = group % kBStages, b_phase = 0;
    bool alive = true;
    for (uint32_t unit = pair; unit < units; unit += pairs) {
      const uint32_t row = ((unit % tiles) / tiles_m) * kBlockN + rank * kHalfN + thread;
      const __half* row_scales = scales + static_cast<size_t>(row) * groups_k + (unit / tiles) * unit_groups;
      for (uint32_t kt = group; kt < k_tiles; kt += kConverterGroups) {
        const uint32_t scale_group = kt / 2u;
        if (scale_group % kChapterGroups == 0u) {
          // Rows past N hold zero codes (TMA fill) and get zero scales; nothing stores them.
          const uint32_t count = min(kChapterGroups, unit_groups - scale_group);
          const __half* source = row_scales + scale_group;
          if (row < n && count % 8u == 0u && (reinterpret_cast<uintptr_t>(source) & 15u) == 0u) {
            for (uint32_t item_group = 0; item_group < count; item_group += 8u) {
              const uint4 eight = __ldg(reinterpret_cast<const uint4*>(source + item_group));
              const uint32_t words[4] = {eight.x, eight.y, eight.z, eight.w};
#pragma unroll
              for (uint32_t item = 0; item < 8u; ++item) {
                store_shared_u16(table + (item_group + item) * (kHalfN * 2u), words[item / 2u] >> (16u * (item % 2u)));
              }
            }
          } else {
            for (uint32_t item = 0; item < count; ++item) {
              store_shared_u16(table + item * (kHalfN * 2u),
                               row < n ? static_cast<uint32_t>(__half_as_ushort(__ldg(source + item))) : 0u);
            }
          }
        }
        // (Once a wait has run out, `abort` is raised and this thread skips every later wait: the
        // loops run to their end on meaningless data and the launch reports the failure.)
        if (alive) alive = ptx::mbarrier_wait<ptx::kWaitBudgetNs, 32u>(&packed_full[packed_stage], packed_phase, abort);
        if (alive) alive = ptx::mbarrier_wait<ptx::kWaitBudgetNs, 32u>(&b_empty[b_stage], b_phase ^ 1u, abort);
        ptx::tcgen05_fence_after();      // the MMAs that read this buffer are behind us
        // This group's 32 bytes of the row's 64 in the packed tile (not swizzled).
        const uint32_t packed_row = ptx::smem_address(shared_packed + packed_stage * L::kPackedBytes) +
                                    thread * 64u + group * 32u;
        const uint32_t b_row = ptx::smem_address(shared_b + b_stage * L::kBBytes) + thread * 128u;
        const uint32_t swizzle = thread % 8u;
        const uint32_t scale2 = load_shared_u16(table + (scale_group % kChapterGroups) * (kHalfN * 2u)) * 0x00010001u;
        const uint4 low = load_shared_16(packed_row);
        const uint4 high = load_shared_16(packed_row + 16u);
        const uint32_t words[8] = {low.x, low.y, low.z, low.w, high.x, high.y, high.z, high.w};
#pragma unroll
        for (uint32_t piece = 0; piece < 8u; ++piece) {
          store_shared_16(b_row + ((piece ^ swizzle) * 16u), expand8(words[piece], scale2));
        }
        // The tensor cores read shared memory through the async proxy: make this thread's stores
        // visible to it, then one arrival per warp on the leader's barrier.
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          ptx::mbarrier_arrive_cluster(ptx::map_to_cta(ptx::smem_address(&converted[b_stage]), 0u));
          // This warp is done with the packed tile (its reads returned before the stores that
          // used them were issued).
          ptx::mbarrier_arrive(&packed_empty[packed_stage]);
        }
        if (++packed_stage == kPackedStages) {
          packed_stage = 0;
          packed_phase ^= 1u;
        }
        // two stages on in the ring of expanded tiles
        b_stage += kConverterGroups;
        if (b_stage >= kBStages) {
          b_stage -= kBStages;
          b_phase ^= 1u;
        }
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

}  // namespace w4a16_pair

namespace w4a16_tile {

int prepare_pair(Config* config) {
  using namespace w4a16_pair;
  int status = static_cast<int>(cudaFuncSetAttribute(w4a16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     Layout::kDynamicBytes));
  if (status != 0) return status;
  // The kernel is persistent: every pair must be resident at once. Not every SM can be paired
  // (it depends on how SMs are grouped on the die), so ask.
  cudaLaunchConfig_t launch_config = {};
  launch_config.gridDim = dim3(static_cast<unsigned int>(config->sm_count) & ~1u, 1, 1);
  launch_config.blockDim = dim3(kThreads, 1, 1);
  launch_config.dynamicSmemBytes = Layout::kDynamicBytes;
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 2;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  launch_config.attrs = &attribute;
  launch_config.numAttrs = 1;
  int clusters = 0;
  status = static_cast<int>(cudaOccupancyMaxActiveClusters(&clusters, w4a16_pair_kernel, &launch_config));
  if (status != 0) return status;
  if (clusters < 1) return static_cast<int>(cudaErrorLaunchOutOfResources);
  config->resident_pairs = clusters;
  return 0;
}

int launch_pair(Config* config, cudaStream_t stream, const void* scales, void* output, void* workspace, int m,
                int n, int k, uint32_t* status_word) {
  using namespace w4a16_pair;
  const uint32_t splits = static_cast<uint32_t>(config->splits);
  const uint32_t units = ((static_cast<uint32_t>(m) + 2u * kBlockM - 1u) / (2u * kBlockM)) *
                         ((static_cast<uint32_t>(n) + kBlockN - 1u) / kBlockN) * splits;
  const uint32_t pairs = units < static_cast<uint32_t>(config->resident_pairs) ? units : config->resident_pairs;
  const uint32_t idesc = ptx::make_f16_idesc(false, 2u * kBlockM, kBlockN);
  return launch_after_dependency(w4a16_pair_kernel, dim3(2u * pairs), dim3(kThreads), Layout::kDynamicBytes, stream,
                                 config->map_a, config->map_w, static_cast<const __half*>(scales),
                                 static_cast<__half*>(output), static_cast<float*>(workspace),
                                 static_cast<uint32_t>(m), static_cast<uint32_t>(n), static_cast<uint32_t>(k),
                                 splits, idesc, status_word);
}

}  // namespace w4a16_tile
}  // namespace mircuda_b200
