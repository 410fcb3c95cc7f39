// int4-g128 W4A16 GEMM for prefill (M > 16): C[M,N] = A[M,K] . dequant(W)[N,K]^T, f16 activations
// and outputs, fp32 accumulation in tensor memory, with the expansion of the 4-bit weights fused
// into the GEMM: the packed weights are read from HBM once per tile and never exist as f16 in
// global memory. (The two-launch form, expansion into an f16 workspace and then the dense GEMM,
// reads and writes that workspace once more per call and took as long for the expansion as for
// the GEMM.)
//
// One persistent 448-thread CTA per SM, tiles of 128 tokens x BN weight rows, 64 K-elements per
// stage:
//  * warp 0 issues the TMA loads: per stage the activation tile (128 rows x 128 bytes, 128-byte
//    swizzle), and once per two stages the packed weight rows of those stages (BN rows x 64
//    bytes);
//  * warps 6-13 (two groups of four taking the stages in turn, two weight rows per thread) turn a
//    row's 32 packed bytes
//    into 64 f16 values (nibble OR-ed into the mantissa of 1024.0, minus 1032 = q - 8 exactly,
//    times the group's f16 scale: the value the two-launch form stores) and write them as the
//    K-major, 128-byte-swizzled B tile the tensor core reads: 16-byte piece c of row r goes to
//    r * 128 + ((c ^ (r % 8)) * 16);
//  * warp 1 issues four tcgen05.mma (kind::f16) per stage once both operands are in place;
//  * warps 2-5 drain the accumulator (32 columns at a time) to f16 outputs.
// When M and N give fewer tiles than half the SMs (M = 256 x N = 4096 is 32 tiles), K is cut
// into `splits` ranges, a unit being (tile, range): the units store fp32 partial tiles into a
// plan-owned workspace and a second small kernel adds the ranges in order and writes f16.
// Every mbarrier wait is bounded; a wait that gives up raises the CTA's abort flag, every role
// leaves its loop, tensor memory is freed and *status is set.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "launch_overlap.hpp"
#include "ptx.cuh"
#include "tensor_map.hpp"
#include "w4a16_expand.cuh"
#include "w4a16_tile.hpp"

namespace mircuda_b200 {
namespace w4a16_tile {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kBlockK = 64;           // K-elements per stage: 128 bytes of f16, 32 of int4
constexpr uint32_t kGroupK = 128;          // elements per scale group: two stages
constexpr uint32_t kConverterThreads = 256;
constexpr uint32_t kThreads = 6u * 32u + kConverterThreads;   // 448
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kChapterGroups = 16;    // scale groups of a row kept in shared memory at a time
constexpr uint32_t kConverterGroups = 2;   // groups of converter warps, taking the stages in turn
constexpr uint32_t kGroupThreads = kConverterThreads / kConverterGroups;   // 128

// STAGES: ring of activation tiles (16 KB each), deep enough to cover the latency of the loads;
// B_STAGES: ring of expanded weight tiles (32 KB each at BN = 256): with two, a tile could only
// be expanded after the MMAs two stages back had finished and the hand-over latencies added up
// to a stage period of twice the MMA time; three let the converters run ahead. kPackedStages:
// ring of packed weight tiles, each the rows' bytes of two stages (16 KB).
constexpr uint32_t kPackedStages = 2;
constexpr uint32_t kQuad = 2;              // stages covered by one packed tile

template <uint32_t BN, uint32_t STAGES, uint32_t B_STAGES>
struct Layout {
  static constexpr uint32_t kAccStages = 2;
  static constexpr uint32_t kABytes = kBlockM * 128u;
  static constexpr uint32_t kBBytes = BN * 128u;
  static constexpr uint32_t kPackedBytes = BN * 32u * kQuad;
  static constexpr uint32_t kBOffset = STAGES * kABytes;
  static constexpr uint32_t kPackedOffset = kBOffset + B_STAGES * kBBytes;
  static constexpr uint32_t kScaleOffset = kPackedOffset + kPackedStages * kPackedBytes;   // [group][row] f16
  static constexpr uint32_t kBarrierOffset = kScaleOffset + kConverterGroups * kChapterGroups * BN * 2u;
  static constexpr uint32_t kBarriers = 2 * STAGES + 2 * B_STAGES + 2 * kPackedStages + 2 * kAccStages;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  static constexpr uint32_t kDynamicBytes = kMiscOffset + 16 + 1024;
  static_assert(kAccStages * BN <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

using namespace w4a16_expand;

template <uint32_t BN, uint32_t STAGES, uint32_t B_STAGES>
__global__ void __launch_bounds__(kThreads, 1)
w4a16_tile_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                  const __half* __restrict__ scales, __half* __restrict__ c, float* __restrict__ partial,
                  uint32_t m, uint32_t n, uint32_t k, uint32_t splits, uint32_t idesc,
                  uint32_t* __restrict__ status) {
  using L = Layout<BN, STAGES, B_STAGES>;
  constexpr uint32_t kAccStages = L::kAccStages;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_a = shared;
  uint8_t* shared_b = shared + L::kBOffset;
  uint8_t* shared_packed = shared + L::kPackedOffset;
  uint64_t* loaded = reinterpret_cast<uint64_t*>(shared + L::kBarrierOffset);   // TMA -> MMA (activations)
  uint64_t* empty = loaded + STAGES;                                             // MMA -> TMA
  uint64_t* converted = empty + STAGES;                                          // converters -> MMA
  uint64_t* b_empty = converted + B_STAGES;                                      // MMA -> converters
  uint64_t* packed_full = b_empty + B_STAGES;                                    // TMA -> converters
  uint64_t* packed_empty = packed_full + kPackedStages;                          // converters -> TMA
  uint64_t* acc_full = packed_empty + kPackedStages;
  uint64_t* acc_empty = acc_full + kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(shared + L::kMiscOffset);
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const uint32_t warp = threadIdx.x / 32u;
  const uint32_t lane = threadIdx.x % 32u;

  if (threadIdx.x == 0) {
    for (uint32_t stage = 0; stage < STAGES; ++stage) {
      ptx::mbarrier_init(&loaded[stage], 1);
      ptx::mbarrier_init(&empty[stage], 1);
    }
    for (uint32_t stage = 0; stage < B_STAGES; ++stage) {
      ptx::mbarrier_init(&converted[stage], kGroupThreads / 32u);
      ptx::mbarrier_init(&b_empty[stage], 1);
    }
    for (uint32_t stage = 0; stage < kPackedStages; ++stage) {
      ptx::mbarrier_init(&packed_full[stage], 1);
      ptx::mbarrier_init(&packed_empty[stage], kConverterThreads / 32u);
    }
    for (uint32_t stage = 0; stage < kAccStages; ++stage) {
      ptx::mbarrier_init(&acc_full[stage], 1);
      ptx::mbarrier_init(&acc_empty[stage], 4);
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&map_a);
    ptx::prefetch_tensor_map(&map_w);
  }
  if (warp == 1) {
    ptx::tmem_allocate(tmem_slot, kTmemColumns);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Nothing above touched global memory; the rest runs after the kernel before this one.
  ptx::dependency_launch_next();
  ptx::dependency_wait();

  const uint32_t tiles_m = (m + kBlockM - 1u) / kBlockM;
  const uint32_t tiles_n = (n + BN - 1u) / BN;
  const uint32_t tiles = tiles_m * tiles_n;
  const uint32_t units = tiles * splits;             // unit = tile + split * tiles
  const uint32_t k_tiles = k / kBlockK / splits;     // per unit (an even number: whole scale groups)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0, packed_stage = 0, packed_phase = 0;
      bool running = true;
      for (uint32_t unit = blockIdx.x; running && unit < units; unit += gridDim.x) {
        const uint32_t tile = unit % tiles;
        const uint32_t first_kt = (unit / tiles) * k_tiles;
        const uint32_t m0 = (tile % tiles_m) * kBlockM;
        const uint32_t n0 = (tile / tiles_m) * BN;
        for (uint32_t kt = first_kt; kt < first_kt + k_tiles; ++kt) {
          if ((kt - first_kt) % kQuad == 0u) {
            // The packed bytes of the next two stages.
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
          ptx::mbarrier_arrive_expect_tx(&loaded[stage], L::kABytes);
          ptx::tma_load_2d(shared_a + stage * L::kABytes, &map_a, &loaded[stage],
                           static_cast<int32_t>(kt * kBlockK), static_cast<int32_t>(m0));
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
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0, b_stage = 0, b_phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      for (uint32_t unit = blockIdx.x; running && unit < units; unit += gridDim.x) {
        if (!ptx::mbarrier_wait<ptx::kWaitBudgetNs, 64u>(&acc_empty[acc_stage], acc_phase ^ 1u, abort)) break;
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * BN;
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
            ptx::mma_f16(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc, (kt | kb) != 0u);
          }
          // These MMAs were the last readers of the stage's activation tile and of the expanded
          // weight tile (its packed source was consumed before them).
          ptx::tcgen05_commit(&empty[stage]);
          ptx::tcgen05_commit(&b_empty[b_stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
          if (++b_stage == B_STAGES) {
            b_stage = 0;
            b_phase ^= 1u;
          }
        }
        if (!running) break;
        ptx::tcgen05_commit(&acc_full[acc_stage]);
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
    for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const uint32_t tile = unit % tiles;
      const uint32_t m0 = (tile % tiles_m) * kBlockM;
      const uint32_t n0 = (tile / tiles_m) * BN;
      float* partial_rows = partial + static_cast<size_t>(unit / tiles) * m * n;
      // The epilogue warps wait for a whole tile's main loop beside the converters: sleep between polls.
      if (!ptx::mbarrier_wait<ptx::kWaitBudgetNs, 256u>(&acc_full[acc_stage], acc_phase, abort)) break;
      ptx::tcgen05_fence_after();
      const uint32_t row = m0 + quarter * 32u + lane;
      const uint32_t tmem_row = tmem_base + ((quarter * 32u) << 16) + acc_stage * BN;
#pragma unroll 1
      for (uint32_t chunk = 0; chunk < BN / 32u; ++chunk) {
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
              for (uint32_t pair = 0; pair < 4u; ++pair) {
                const __half2 two = __floats2half2_rn(__uint_as_float(values[part * 8u + pair * 2u]),
                                                      __uint_as_float(values[part * 8u + pair * 2u + 1u]));
                packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
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
      if (lane == 0) ptx::mbarrier_arrive(&acc_empty[acc_stage]);
      if (++acc_stage == kAccStages) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ converters
    // Two groups of four warps take the stages in turn (group g the stages with kt % 2 == g, a
    // thread the rows t and t + 128 of the tile), so that two stages are being expanded at any
    // time: one stage's expansion is a chain of shared-memory loads, arithmetic, stores and a
    // proxy fence about as long as two stages of MMAs, and a single group working stage after
    // stage held the tensor pipe at a third of its rate.
    static_assert(BN == 2u * kGroupThreads, "two weight rows per converter thread");
    static_assert(kQuad == kConverterGroups, "every group takes one stage of a packed tile");
    const uint32_t group = (threadIdx.x - 6u * 32u) / kGroupThreads;
    const uint32_t thread = (threadIdx.x - 6u * 32u) % kGroupThreads;
    const uint32_t groups_k = k / kGroupK;
    const uint32_t unit_groups = k_tiles / 2u;
    // The rows' scales of the next kChapterGroups scale groups live in shared memory, one table
    // per converter group, [scale group][row] so that a warp's reads are adjacent; a thread
    // writes and reads only its own two columns, so no barrier is needed. (Global loads are kept
    // out of the stage loop: the proxy fence at the end of a stage waits for every load the
    // thread still has in flight.)
    const uint32_t table = ptx::smem_address(shared + L::kScaleOffset) + group * (kChapterGroups * BN * 2u) +
                           thread * 2u;
    // Ring positions advance with every stage, also the other group's.
    uint32_t packed_stage = 0, packed_phase = 0, b_stage = group % B_STAGES, b_phase = 0;
    bool alive = true;
    for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const uint32_t first_row = ((unit % tiles) / tiles_m) * BN + thread;
      const __half* unit_scales = scales + (unit / tiles) * unit_groups;
      for (uint32_t kt = group; kt < k_tiles; kt += kConverterGroups) {
        const uint32_t scale_group = kt / 2u;
        if (scale_group % kChapterGroups == 0u) {
          // Rows past N hold zero codes (TMA fill) and get zero scales; nothing stores them.
          const uint32_t count = min(kChapterGroups, unit_groups - scale_group);
#pragma unroll
          for (uint32_t part = 0; part < 2u; ++part) {
            const uint32_t row = first_row + part * kGroupThreads;
            const __half* source = unit_scales + static_cast<size_t>(row) * groups_k + scale_group;
            const uint32_t column = table + part * (kGroupThreads * 2u);
            if (row < n && count % 8u == 0u && (reinterpret_cast<uintptr_t>(source) & 15u) == 0u) {
              for (uint32_t item_group = 0; item_group < count; item_group += 8u) {
                const uint4 eight = __ldg(reinterpret_cast<const uint4*>(source + item_group));
                const uint32_t words[4] = {eight.x, eight.y, eight.z, eight.w};
#pragma unroll
                for (uint32_t item = 0; item < 8u; ++item) {
                  store_shared_u16(column + (item_group + item) * (BN * 2u), words[item / 2u] >> (16u * (item % 2u)));
                }
              }
            } else {
              for (uint32_t item = 0; item < count; ++item) {
                store_shared_u16(column + item * (BN * 2u),
                                 row < n ? static_cast<uint32_t>(__half_as_ushort(__ldg(source + item))) : 0u);
              }
            }
          }
        }
        // (Once a wait has run out, `abort` is raised and this thread skips every later wait: the
        // loops run to their end on meaningless data and the launch reports the failure.)
        if (alive) alive = ptx::mbarrier_wait<ptx::kWaitBudgetNs, 32u>(&packed_full[packed_stage], packed_phase, abort);
        if (alive) alive = ptx::mbarrier_wait<ptx::kWaitBudgetNs, 32u>(&b_empty[b_stage], b_phase ^ 1u, abort);
        ptx::tcgen05_fence_after();      // the MMAs that read this buffer are behind us
        // This group's 32 bytes of a row's 64 in the packed tile (not swizzled).
        const uint32_t packed_tile = ptx::smem_address(shared_packed + packed_stage * L::kPackedBytes) + group * 32u;
        const uint32_t b_tile = ptx::smem_address(shared_b + b_stage * L::kBBytes);
        const uint32_t swizzle = thread % 8u;     // the same for both rows (128 apart)
#pragma unroll
        for (uint32_t part = 0; part < 2u; ++part) {
          const uint32_t row = thread + part * kGroupThreads;
          const uint32_t scale2 = load_shared_u16(table + part * (kGroupThreads * 2u) +
                                                  (scale_group % kChapterGroups) * (BN * 2u)) * 0x00010001u;
          const uint4 low = load_shared_16(packed_tile + row * 64u);
          const uint4 high = load_shared_16(packed_tile + row * 64u + 16u);
          const uint32_t words[8] = {low.x, low.y, low.z, low.w, high.x, high.y, high.z, high.w};
#pragma unroll
          for (uint32_t piece = 0; piece < 8u; ++piece) {
            store_shared_16(b_tile + row * 128u + ((piece ^ swizzle) * 16u), expand8(words[piece], scale2));
          }
        }
        // The tensor core reads shared memory through the async proxy: make this thread's
        // stores visible to it, then one arrival per warp.
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) ptx::mbarrier_arrive(&converted[b_stage]);
        // This warp is done with the packed tile (its reads returned before the stores that used
        // them were issued).
        if (lane == 0) ptx::mbarrier_arrive(&packed_empty[packed_stage]);
        if (++packed_stage == kPackedStages) {
          packed_stage = 0;
          packed_phase ^= 1u;
        }
        // two stages on in the ring of expanded tiles
        b_stage += kConverterGroups;
        if (b_stage >= B_STAGES) {
          b_stage -= B_STAGES;
          b_phase ^= 1u;
        }
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

// Adds the K ranges' fp32 partial results in range order and writes f16; eight outputs a thread.
__global__ void __launch_bounds__(256)
w4a16_reduce_kernel(const float* __restrict__ partial, __half* __restrict__ c, size_t vectors, uint32_t splits) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  for (size_t vector = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; vector < vectors;
       vector += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float sums[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t split = 0; split < splits; ++split) {
      const float4* source = reinterpret_cast<const float4*>(partial) + (split * vectors + vector) * 2u;
      const float4 low = __ldcs(source), high = __ldcs(source + 1);
      sums[0] += low.x;
      sums[1] += low.y;
      sums[2] += low.z;
      sums[3] += low.w;
      sums[4] += high.x;
      sums[5] += high.y;
      sums[6] += high.z;
      sums[7] += high.w;
    }
    uint32_t packed[4];
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
      const __half2 two = __floats2half2_rn(sums[2 * pair], sums[2 * pair + 1]);
      packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
    }
    reinterpret_cast<uint4*>(c)[vector] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

constexpr uint32_t kBlockN = 256;
constexpr uint32_t kStages = 5;
constexpr uint32_t kBStages = 3;

bool eligible(int m, int n, int k) { return m > 0 && n > 0 && n % 8 == 0 && k > 0 && k % kGroupK == 0; }

int prepare(Config* config, int m, int n, int k) {
  if (!eligible(m, n, k)) return -1;
  int device = 0;
  int status = static_cast<int>(cudaGetDevice(&device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&config->sm_count, cudaDevAttrMultiProcessorCount, device));
  }
  if (status == 0) {
    status = static_cast<int>(cudaFuncSetAttribute(w4a16_tile_kernel<kBlockN, kStages, kBStages>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   Layout<kBlockN, kStages, kBStages>::kDynamicBytes));
  }
  if (status != 0) return status;
  // More than 128 tokens run on CTA pairs (tiles of 256 tokens; MIRCUDA_B200_W4A16_PREFILL=single
  // keeps single CTAs).
  const char* choice = std::getenv("MIRCUDA_B200_W4A16_PREFILL");
  config->pair = m > static_cast<int>(kBlockM) && !(choice != nullptr && std::strcmp(choice, "single") == 0);
  config->resident_pairs = 0;
  if (config->pair) {
    status = prepare_pair(config);
    if (status != 0) return status;
  }
  // K ranges: as many as fill the SMs when the tiles alone leave more than half of them idle,
  // each a whole number of scale groups (two stages) and at least eight groups long.
  const int tile_m = static_cast<int>(kBlockM) * (config->pair ? 2 : 1);
  const int slots = config->pair ? config->resident_pairs : config->sm_count;
  const int tiles = ((m + tile_m - 1) / tile_m) * ((n + static_cast<int>(kBlockN) - 1) / static_cast<int>(kBlockN));
  const int groups = k / static_cast<int>(kGroupK);
  int splits = 1;
  if (tiles * 2 <= slots) {
    for (int candidate = slots / tiles; candidate >= 2; --candidate) {
      if (groups % candidate == 0 && groups / candidate >= 8) {
        splits = candidate;
        break;
      }
    }
  }
  config->splits = splits;
  config->workspace_bytes = splits > 1 ? static_cast<size_t>(splits) * m * n * sizeof(float) : 0u;
  config->cached_input = nullptr;
  config->cached_weight = nullptr;
  return 0;
}

int launch(Config* config, cudaStream_t stream, const void* input, const void* weight, const void* scales,
           void* output, void* workspace, int m, int n, int k, uint32_t* status_word) {
  if (config->splits > 1 && workspace == nullptr) return -1;
  if (input != config->cached_input) {
    const int status = encode_k_major_map(&config->map_a, input, m, k, 2u, kBlockM);
    if (status != 0) return status;
    config->cached_input = input;
  }
  if (weight != config->cached_weight) {
    // Packed weights as bytes [N, K / 2]; a box is 64 bytes (two stages' codes) of BN rows.
    EncodeTiled encode = encode_tiled_entry();
    if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
    const cuuint64_t dimensions[2] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k / 2)};
    const cuuint32_t box[2] = {kQuad * kBlockK / 2u, config->pair ? kBlockN / 2u : kBlockN};
    const cuuint32_t element_strides[2] = {1u, 1u};
    const int status = static_cast<int>(encode(
        &config->map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2u, const_cast<void*>(weight), dimensions, strides, box,
        element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    if (status != 0) return status;
    config->cached_weight = weight;
  }
  const uint32_t splits = static_cast<uint32_t>(config->splits);
  int status = 0;
  if (config->pair) {
    status = launch_pair(config, stream, scales, output, workspace, m, n, k, status_word);
  } else {
    const uint32_t units = ((static_cast<uint32_t>(m) + kBlockM - 1u) / kBlockM) *
                           ((static_cast<uint32_t>(n) + kBlockN - 1u) / kBlockN) * splits;
    const uint32_t grid = units < static_cast<uint32_t>(config->sm_count) ? units : config->sm_count;
    const uint32_t idesc = ptx::make_f16_idesc(false, kBlockM, kBlockN);
    status = launch_after_dependency(w4a16_tile_kernel<kBlockN, kStages, kBStages>, dim3(grid), dim3(kThreads),
                                     Layout<kBlockN, kStages, kBStages>::kDynamicBytes, stream, config->map_a,
                                     config->map_w, static_cast<const __half*>(scales),
                                     static_cast<__half*>(output), static_cast<float*>(workspace),
                                     static_cast<uint32_t>(m), static_cast<uint32_t>(n),
                                     static_cast<uint32_t>(k), splits, idesc, status_word);
  }
  if (status == 0 && splits > 1u) {
    const size_t vectors = static_cast<size_t>(m) * n / 8u;
    const size_t blocks = (vectors + 255u) / 256u;
    status = launch_after_dependency(w4a16_reduce_kernel,
                                     dim3(static_cast<unsigned int>(blocks < 148u * 16u ? blocks : 148u * 16u)),
                                     dim3(256), 0, stream, static_cast<const float*>(workspace),
                                     static_cast<__half*>(output), vectors, splits);
  }
  return status;
}

}  // namespace w4a16_tile
}  // namespace mircuda_b200
