// Variable-row grouped bf16 GEMM for MoE layers on sm_100a. For each group g the rows
// [offsets[g], offsets[g] + min(rows[g], max_rows)) of the compact activation matrix
// A[capacity, K] are multiplied by that group's weight W_g[N, K]^T into the same rows of
// C[capacity, N] (fp32 accumulation in tensor memory, C = acc + beta * C, bf16 out).
// Replaces the reference's CUTLASS grouped kernel (sys/native/variable_grouped_bf16_sm120.cu,
// mma.sync tiles with a device-side problem visitor) behind the same C entry points. Row
// counts and offsets stay on the device: a small set-up kernel turns them into a running
// count of 128-row tiles per group, and the persistent main kernel maps its linear tile index
// to (group, row tile, column tile) by binary search, groups outermost so that CTAs running
// together share one group's weights in L2.
//
// Main kernel structure (192 threads, one CTA per SM): warp 0 issues TMA loads (A by a 2-D
// map over the compact rows, B by a 3-D map [G, N, K]; both 128-byte-swizzled K-major tiles
// of 64 bf16), warp 1 issues tcgen05.mma.kind::f16 (four K=16 steps per stage), warps 2-5
// drain the accumulator. A group's last row tile is ragged and the rows after it belong to
// the next group or lie past the buffer, so it is loaded as power-of-two row pieces
// (64, 32, ... 1 rows, one tensor map per piece size): nothing outside the group's rows is
// ever read, and stores are predicated per row. Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <new>

#include "launch_overlap.hpp"
#include "ptx.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace grouped_bf16 {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kBlockKBytes = 128;     // 64 bf16 per stage row
constexpr uint32_t kBlockK = 64;
constexpr uint32_t kThreads = 192;
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kPieceMaps = 8;         // A tensor maps with box rows 128, 64, ..., 1

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
struct Layout {
  static constexpr uint32_t kABytes = kBlockM * kBlockKBytes;
  static constexpr uint32_t kBBytes = BN * kBlockKBytes;
  static constexpr uint32_t kBOffset = STAGES * kABytes;
  static constexpr uint32_t kBarrierOffset = kBOffset + STAGES * kBBytes;
  static constexpr uint32_t kBarriers = 2 * STAGES + 2 * ACC_STAGES;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  // Tile starts of up to kSharedGroups groups, copied once per CTA: the per-tile binary search
  // then runs on shared memory instead of on a chain of dependent L2 round trips.
  static constexpr uint32_t kSharedGroups = 2048;
  static constexpr uint32_t kStartsOffset = kMiscOffset + 16;
  static constexpr uint32_t kDynamicBytes = kStartsOffset + (kSharedGroups + 1) * 4 + 1024;
  static_assert(ACC_STAGES * BN <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

struct MapSet {
  CUtensorMap a[kPieceMaps];   // box rows 128 >> index
  CUtensorMap b;
};

// tile_starts[g] = number of tiles in groups before g (tiles = row tiles x column tiles);
// tile_starts[groups] = total. One block; a serial carry across 1024-wide chunks.
__global__ void __launch_bounds__(1024)
grouped_bf16_setup_kernel(const unsigned int* __restrict__ rows,
                          const unsigned int* __restrict__ indices, uint32_t matrices,
                          uint32_t groups, uint32_t max_rows, uint32_t tiles_n,
                          uint32_t* __restrict__ tile_starts) {
  __shared__ uint32_t warp_totals[32];
  __shared__ uint32_t carry;
  // The routing arrays come from the kernel before this one; the main kernel after this one may
  // set itself up meanwhile.
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  if (threadIdx.x == 0) carry = 0u;
  __syncthreads();
  for (uint32_t base = 0; base < groups; base += 1024u) {
    const uint32_t group = base + threadIdx.x;
    uint32_t count = 0u;
    if (group < groups) {
      // A group whose matrix index is out of range gets no tiles (it is skipped).
      const bool routed = indices == nullptr || indices[group] < matrices;
      const uint32_t row_count = routed ? min(rows[group], max_rows) : 0u;
      count = ((row_count + kBlockM - 1u) / kBlockM) * tiles_n;
    }
    uint32_t inclusive = count;
#pragma unroll
    for (uint32_t offset = 1; offset < 32u; offset <<= 1) {
      const uint32_t other = __shfl_up_sync(0xffffffffu, inclusive, offset);
      if ((threadIdx.x & 31u) >= offset) inclusive += other;
    }
    if ((threadIdx.x & 31u) == 31u) warp_totals[threadIdx.x >> 5] = inclusive;
    __syncthreads();
    if (threadIdx.x < 32u) {
      uint32_t total = warp_totals[threadIdx.x];
#pragma unroll
      for (uint32_t offset = 1; offset < 32u; offset <<= 1) {
        const uint32_t other = __shfl_up_sync(0xffffffffu, total, offset);
        if (threadIdx.x >= offset) total += other;
      }
      warp_totals[threadIdx.x] = total;
    }
    __syncthreads();
    const uint32_t before_warp = (threadIdx.x >> 5) == 0u ? 0u : warp_totals[(threadIdx.x >> 5) - 1u];
    const uint32_t exclusive = carry + before_warp + inclusive - count;
    if (group < groups) tile_starts[group] = exclusive;
    __syncthreads();
    if (threadIdx.x == 1023u) carry = exclusive + count;
    __syncthreads();
  }
  if (threadIdx.x == 0) tile_starts[groups] = carry;
}

struct Tile {
  uint32_t group;
  uint32_t row0;        // first row in the compact matrices
  uint32_t valid_rows;  // 1..128
  uint32_t n0;
};

// Linear tile index -> tile. Inside a group, row tiles vary fastest.
// `starts` is the shared-memory copy of tile_starts when the groups fit, else the global array.
__device__ __forceinline__ Tile locate(uint32_t index, const uint32_t* starts,
                                       const unsigned int* __restrict__ rows,
                                       const unsigned int* __restrict__ offsets, uint32_t groups,
                                       uint32_t max_rows, uint32_t block_n) {
  uint32_t low = 0u, high = groups;       // last group whose start is <= index
  while (high - low > 1u) {
    const uint32_t middle = (low + high) / 2u;
    if (starts[middle] <= index) low = middle; else high = middle;
  }
  // Groups without tiles share their start with the next group; step past them.
  while (low + 1u < groups && starts[low + 1u] <= index) ++low;
  const uint32_t row_count = min(__ldg(rows + low), max_rows);
  const uint32_t row_tiles = (row_count + kBlockM - 1u) / kBlockM;
  const uint32_t local = index - starts[low];
  const uint32_t row_tile = local % row_tiles;
  Tile tile;
  tile.group = low;
  tile.row0 = __ldg(offsets + low) + row_tile * kBlockM;
  tile.valid_rows = min(kBlockM, row_count - row_tile * kBlockM);
  tile.n0 = (local / row_tiles) * block_n;
  return tile;
}

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
__global__ void __launch_bounds__(kThreads, 1)
grouped_bf16_kernel(const __grid_constant__ MapSet maps, const unsigned int* __restrict__ rows,
                    const unsigned int* __restrict__ offsets,
                    const unsigned int* __restrict__ indices,
                    const uint32_t* __restrict__ tile_starts, __nv_bfloat16* __restrict__ c,
                    uint32_t groups, uint32_t max_rows, uint32_t n, uint32_t k, float beta,
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
    ptx::prefetch_tensor_map(&maps.a[0]);
    ptx::prefetch_tensor_map(&maps.b);
  }
  if (warp == 1) {
    ptx::tmem_allocate(tmem_slot, kTmemColumns);
    ptx::tmem_relinquish();
  }
  // Barriers, tensor memory and the tensor-map prefetch above needed nothing from global memory
  // and may have run beside the set-up kernel; its tile starts are read from here on.
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  uint32_t* starts_table = reinterpret_cast<uint32_t*>(shared + L::kStartsOffset);
  const uint32_t* starts = tile_starts;
  if (groups <= L::kSharedGroups) {
    for (uint32_t group = threadIdx.x; group <= groups; group += kThreads) {
      starts_table[group] = __ldg(tile_starts + group);
    }
    starts = starts_table;
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t tiles = __ldg(tile_starts + groups);
  const uint32_t k_tiles = (k + kBlockK - 1u) / kBlockK;

  if (warp == 0) {
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool running = true;
      // The next tile's routing is fetched while this tile's loads are being issued.
      Tile upcoming = {};
      uint32_t upcoming_matrix = 0u;
      if (blockIdx.x < tiles) {
        upcoming = locate(blockIdx.x, starts, rows, offsets, groups, max_rows, BN);
        upcoming_matrix = indices == nullptr ? upcoming.group : __ldg(indices + upcoming.group);
      }
      for (uint32_t index = blockIdx.x; running && index < tiles; index += gridDim.x) {
        const Tile tile = upcoming;
        const uint32_t matrix = upcoming_matrix;
        if (index + gridDim.x < tiles) {
          upcoming = locate(index + gridDim.x, starts, rows, offsets, groups, max_rows, BN);
          upcoming_matrix = indices == nullptr ? upcoming.group : __ldg(indices + upcoming.group);
        }
        for (uint32_t kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          ptx::mbarrier_arrive_expect_tx(&full[stage],
                                         tile.valid_rows * kBlockKBytes + L::kBBytes);
          uint8_t* a_stage = shared_a + stage * L::kABytes;
          const int32_t x = static_cast<int32_t>(kt * kBlockK);
          if (tile.valid_rows == kBlockM) {
            ptx::tma_load_2d(a_stage, &maps.a[0], &full[stage], x,
                             static_cast<int32_t>(tile.row0));
          } else {
            // Ragged last tile of a group: pieces of 64, 32, ... 1 rows. A piece of p rows
            // starts at a multiple of p rows, so pieces of 8 or more rows start on the
            // 1024-byte swizzle period and smaller ones keep their place inside it.
            uint32_t done = 0u;
#pragma unroll
            for (uint32_t piece = 1; piece < kPieceMaps; ++piece) {
              const uint32_t piece_rows = kBlockM >> piece;
              if ((tile.valid_rows & piece_rows) != 0u) {
                ptx::tma_load_2d(a_stage + done * kBlockKBytes, &maps.a[piece], &full[stage], x,
                                 static_cast<int32_t>(tile.row0 + done));
                done += piece_rows;
              }
            }
          }
          ptx::tma_load_3d(shared_b + stage * L::kBBytes, &maps.b, &full[stage], x,
                           static_cast<int32_t>(tile.n0), static_cast<int32_t>(matrix));
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
      constexpr uint32_t idesc = ptx::make_f16_idesc(true, kBlockM, BN);
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      for (uint32_t index = blockIdx.x; running && index < tiles; index += gridDim.x) {
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
    // 32-byte stores need rows that start on 32-byte boundaries
    const bool wide_stores = (n % 16u) == 0u && (reinterpret_cast<uintptr_t>(c) & 31u) == 0u;
    for (uint32_t index = blockIdx.x; index < tiles; index += gridDim.x) {
      const Tile tile = locate(index, starts, rows, offsets, groups, max_rows, BN);
      if (!ptx::mbarrier_wait(&acc_full[acc_stage], acc_phase, abort)) break;
      ptx::tcgen05_fence_after();
      const uint32_t row_in_tile = quarter * 32u + lane;
      const uint32_t tmem_row = tmem_base + ((quarter * 32u) << 16) + acc_stage * BN;
      const bool row_valid = row_in_tile < tile.valid_rows;
      __nv_bfloat16* c_row = c + static_cast<size_t>(tile.row0 + row_in_tile) * n;
#pragma unroll 1
      for (uint32_t chunk = 0; chunk < BN / 32u; ++chunk) {
        uint32_t values[32];
        ptx::tmem_load_32x32(tmem_row + chunk * 32u, values);
        ptx::tmem_load_wait();
        const uint32_t column = tile.n0 + chunk * 32u;
        if (row_valid && column < n) {
          __nv_bfloat16* destination = c_row + column;
          if (column + 32u <= n) {
            uint32_t packed[16];
#pragma unroll
            for (uint32_t part = 0; part < 4u; ++part) {
              float v[8];
#pragma unroll
              for (uint32_t item = 0; item < 8u; ++item) v[item] = __uint_as_float(values[part * 8u + item]);
              if (beta != 0.0f) {
                const uint4 previous = reinterpret_cast<const uint4*>(destination)[part];
                const uint32_t words[4] = {previous.x, previous.y, previous.z, previous.w};
#pragma unroll
                for (uint32_t pair = 0; pair < 4u; ++pair) {
                  v[pair * 2u] = fmaf(beta, __uint_as_float(words[pair] << 16), v[pair * 2u]);
                  v[pair * 2u + 1u] =
                      fmaf(beta, __uint_as_float(words[pair] & 0xffff0000u), v[pair * 2u + 1u]);
                }
              }
#pragma unroll
              for (uint32_t pair = 0; pair < 4u; ++pair) {
                const __nv_bfloat162 two = __floats2bfloat162_rn(v[pair * 2u], v[pair * 2u + 1u]);
                packed[part * 4u + pair] = *reinterpret_cast<const uint32_t*>(&two);
              }
            }
            if (wide_stores) {
              // 32 bytes per store fill whole sectors; 16-byte stores to the same rows cost twice
              // the L1 -> L2 write traffic.
#pragma unroll
              for (uint32_t half = 0; half < 2u; ++half) {
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(destination + half * 16u),
                             "r"(packed[half * 8u + 0u]), "r"(packed[half * 8u + 1u]), "r"(packed[half * 8u + 2u]),
                             "r"(packed[half * 8u + 3u]), "r"(packed[half * 8u + 4u]), "r"(packed[half * 8u + 5u]),
                             "r"(packed[half * 8u + 6u]), "r"(packed[half * 8u + 7u])
                             : "memory");
              }
            } else {
#pragma unroll
              for (uint32_t part = 0; part < 4u; ++part) {
                reinterpret_cast<uint4*>(destination)[part] =
                    make_uint4(packed[part * 4u], packed[part * 4u + 1u], packed[part * 4u + 2u], packed[part * 4u + 3u]);
              }
            }
          } else {
#pragma unroll
            for (uint32_t item = 0; item < 32u; ++item) {
              if (column + item < n) {
                float value = __uint_as_float(values[item]);
                if (beta != 0.0f) value = fmaf(beta, __bfloat162float(destination[item]), value);
                destination[item] = __float2bfloat16_rn(value);
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
  int groups, max_rows, n, k;
  int matrices;              // weight matrices in the bank (== groups without indices)
  int device, sm_count;
  uint32_t block_n;
  cudaStream_t stream;
  uint32_t* tile_starts;     // device, groups + 1 entries
  uint32_t* status;          // pinned
  const void* cached_input;
  const void* cached_weights;
  MapSet maps;
};

inline int encode_3d_weight_map(CUtensorMap* map, const void* base, uint64_t groups, uint64_t n,
                                uint64_t k, uint32_t box_rows) {
  EncodeTiled encode = encode_tiled_entry();
  if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dimensions[3] = {k, n, groups};
  const cuuint64_t strides[2] = {k * 2u, n * k * 2u};
  const cuuint32_t box[3] = {kBlockK, box_rows, 1u};
  const cuuint32_t element_strides[3] = {1u, 1u, 1u};
  return static_cast<int>(encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3u, const_cast<void*>(base),
                                 dimensions, strides, box, element_strides,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
}

template <uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
int launch(Plan* plan, const unsigned int* rows, const unsigned int* offsets,
           const unsigned int* indices, void* c, float beta) {
  using L = Layout<BN, STAGES, ACC_STAGES>;
  auto function = grouped_bf16_kernel<BN, STAGES, ACC_STAGES>;
  static thread_local int configured_device = -1;
  if (configured_device != plan->device) {
    const int status = static_cast<int>(cudaFuncSetAttribute(
        function, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
    if (status != 0) return status;
    configured_device = plan->device;
  }
  return launch_after_dependency(function, dim3(plan->sm_count), dim3(kThreads), L::kDynamicBytes, plan->stream,
                                 plan->maps, rows, offsets, indices, plan->tile_starts,
                                 static_cast<__nv_bfloat16*>(c), static_cast<uint32_t>(plan->groups),
                                 static_cast<uint32_t>(plan->max_rows), static_cast<uint32_t>(plan->n),
                                 static_cast<uint32_t>(plan->k), beta, plan->status);
}

}  // namespace grouped_bf16
}  // namespace mircuda_b200

namespace mircuda_b200 {
namespace grouped_bf16 {

int create(int groups, int matrices, int max_rows, int n, int k, void* stream, void** output) {
  if (groups <= 0 || matrices <= 0 || max_rows <= 0 || n <= 0 || k <= 0 || n % 8 != 0 ||
      k % 8 != 0 || stream == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->groups = groups;
  plan->matrices = matrices;
  plan->max_rows = max_rows;
  plan->n = n;
  plan->k = k;
  plan->stream = static_cast<cudaStream_t>(stream);
  plan->block_n = 256u;
  if (const char* forced = std::getenv("MIRCUDA_B200_GROUPED_BN")) {
    const int value = std::atoi(forced);
    if (value == 128 || value == 256) plan->block_n = static_cast<uint32_t>(value);
  } else if (n <= 128) {
    plan->block_n = 128u;
  }
  int status = static_cast<int>(cudaGetDevice(&plan->device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&plan->sm_count,
                                                     cudaDevAttrMultiProcessorCount, plan->device));
  }
  if (status == 0) {
    status = static_cast<int>(cudaMallocAsync(reinterpret_cast<void**>(&plan->tile_starts),
                                              (static_cast<size_t>(groups) + 1u) * sizeof(uint32_t),
                                              plan->stream));
  }
  if (status == 0) {
    status = static_cast<int>(cudaHostAlloc(reinterpret_cast<void**>(&plan->status),
                                            sizeof(uint32_t), cudaHostAllocMapped));
  }
  if (status != 0) {
    if (plan->tile_starts != nullptr) cudaFreeAsync(plan->tile_starts, plan->stream);
    delete plan;
    return status;
  }
  *plan->status = 0u;
  *output = plan;
  return 0;
}

int execute(void* raw, void* stream, const void* input, const void* weights,
            const unsigned int* indices, const unsigned int* rows, const unsigned int* offsets,
            void* output, float beta) {
  if (raw == nullptr || stream == nullptr || input == nullptr || weights == nullptr ||
      rows == nullptr || offsets == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  if (((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(weights) |
        reinterpret_cast<uintptr_t>(output)) & 15u) != 0u) {
    return -1;
  }
  if (input != plan->cached_input) {
    // The row extent of the compact matrix is not part of this interface; loads are issued
    // only for rows a group owns, so the map's row bound is left wide open.
    for (uint32_t piece = 0; piece < kPieceMaps; ++piece) {
      const int status = encode_k_major_map(&plan->maps.a[piece], input, 0x7fffffffull,
                                            static_cast<uint64_t>(plan->k), 2u, kBlockM >> piece);
      if (status != 0) return status;
    }
    plan->cached_input = input;
  }
  if (weights != plan->cached_weights) {
    const int status = encode_3d_weight_map(&plan->maps.b, weights, plan->matrices, plan->n,
                                            plan->k, plan->block_n);
    if (status != 0) return status;
    plan->cached_weights = weights;
  }
  const uint32_t tiles_n = (plan->n + plan->block_n - 1u) / plan->block_n;
  int status = launch_after_dependency(grouped_bf16_setup_kernel, dim3(1), dim3(1024), 0, cuda_stream, rows,
                                       indices, static_cast<uint32_t>(plan->matrices),
                                       static_cast<uint32_t>(plan->groups),
                                       static_cast<uint32_t>(plan->max_rows), tiles_n, plan->tile_starts);
  if (status != 0) return status;
  return plan->block_n == 128u ? launch<128u, 6u, 4u>(plan, rows, offsets, indices, output, beta)
                               : launch<256u, 4u, 2u>(plan, rows, offsets, indices, output, beta);
}

}  // namespace grouped_bf16
}  // namespace mircuda_b200

extern "C" int mircuda_variable_grouped_bf16_create(int groups, int max_rows, int n, int k,
                                                    void* stream, void** output) {
  return mircuda_b200::grouped_bf16::create(groups, groups, max_rows, n, k, stream, output);
}

extern "C" int mircuda_variable_grouped_bf16_execute(void* raw, void* stream, const void* input,
                                                     const void* weights,
                                                     const unsigned int* rows,
                                                     const unsigned int* offsets, void* output,
                                                     float beta) {
  return mircuda_b200::grouped_bf16::execute(raw, stream, input, weights, nullptr, rows, offsets,
                                             output, beta);
}

extern "C" int mircuda_b200_variable_grouped_bf16_create_indexed(int groups, int matrices,
                                                                 int max_rows, int n, int k,
                                                                 void* stream, void** output) {
  return mircuda_b200::grouped_bf16::create(groups, matrices, max_rows, n, k, stream, output);
}

extern "C" int mircuda_b200_variable_grouped_bf16_execute_indexed(
    void* raw, void* stream, const void* input, const void* weights, const unsigned int* indices,
    const unsigned int* rows, const unsigned int* offsets, void* output, float beta) {
  if (indices == nullptr) return -1;
  return mircuda_b200::grouped_bf16::execute(raw, stream, input, weights, indices, rows, offsets,
                                             output, beta);
}

extern "C" void mircuda_variable_grouped_bf16_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::grouped_bf16::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->tile_starts != nullptr) cudaFreeAsync(plan->tile_starts, plan->stream);
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
