// Grouped NVFP4 block-scaled GEMMs for MoE layers on sm_100a, three entry-point families
// over one kernel:
//   mircuda_variable_grouped_fp4_*          variable rows per group, matrix picked by indices[g]
//   mircuda_paired_variable_grouped_fp4_*   two such problems (e.g. gate and up) sharing routing
//   mircuda_grouped_fp4_*                   fixed m rows per group (decode), optional broadcast input
// For group g with matrix j = indices[g] (groups whose j is out of range are skipped):
//   C[c_row + r, :] = bf16(alphas[j] * sum_k e2m1(A[a_row + r, k]) * ue4m3(SA) * e2m1(B_j[:, k]) * ue4m3(SB))
// A [capacity, K/2] and B [matrices, N, K/2] hold two E2M1 codes per byte (even k low); the
// scales are UE4M3 bytes per 16 K-elements in 512-byte atoms of 128 rows x 4 columns. A's
// scale atoms are addressed per group: a group's row r lives in row tile
// scale_offsets[g] / 128 + r / 128 (the reference's layout,
// sys/native/variable_grouped_fp4_sm120.cu:31-62, grouped_fp4_sm120.cu:29-57; it replaces
// those CUTLASS Sm120 ping-pong kernels behind the same C entry points).
//
// A set-up kernel turns the device-resident routing into one record per group and a running
// count of 128-row x 128-column tiles; the persistent main kernel (192 threads, one CTA per
// SM) maps its linear tile index to (problem side, group, row tile, column tile) by binary
// search. Warp 0 issues TMA loads per 256-element K stage: A [128 x 128 B] (a group's ragged
// last tile as power-of-two row pieces, so nothing outside the group's rows is read), B by a
// 3-D map over the matrices, and the four scale atoms of each operand by flat 2 KB bulk
// copies; warp 1 copies the scales into tensor memory (one 32-column buffer per stage) and
// issues four tcgen05.mma.kind::mxf4nvf4.block_scale.block16 (K = 64 each); warps 2-5 drain
// the accumulator, apply alpha and store row-predicated bf16. Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <new>

#include "launch_overlap.hpp"
#include "layout.cuh"
#include "nvfp4_block.cuh"
#include "ptx.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace grouped_fp4 {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kStageBytesK = 128;     // 256 E2M1 codes per stage row
constexpr uint32_t kStageElements = 256;
constexpr uint32_t kAtomBytes = 512;
constexpr uint32_t kAtomsK = 4;            // scale atoms (64 K-elements each) per stage
// Warps: TMA producer, MMA issuer, then one or two sets of four epilogue warps (a warp reads the
// tensor-memory lanes of quarter warp % 4; two sets split a tile's columns between them).
constexpr uint32_t threads_for(uint32_t epilogue_sets) { return (2u + 4u * epilogue_sets) * 32u; }
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kPieceMaps = 8;         // A tensor maps with box rows 128, 64, ..., 1

// Tile width BN: 128 (two accumulators in tensor memory, six stages; the default) or 256 (one
// accumulator, four stages). The wide tile reads every A tile half as often and halves the
// tile count, but its single accumulator makes the MMAs of the next tile wait for the epilogue.
template <uint32_t BN>
struct Layout {
  static_assert(BN == 128 || BN == 256, "supported tile widths");
  static constexpr uint32_t kStages = BN == 128 ? 6 : 4;
  static constexpr uint32_t kAccStages = BN == 128 ? 2 : 1;
  static constexpr uint32_t kAtomsN = BN / 128;                      // 128-row scale tiles of B per tile
  static constexpr uint32_t kABytes = kBlockM * kStageBytesK;
  static constexpr uint32_t kBBytes = BN * kStageBytesK;
  static constexpr uint32_t kSfaBytes = kAtomsK * kAtomBytes;        // per stage
  static constexpr uint32_t kSfbBytes = kAtomsN * kAtomsK * kAtomBytes;
  static constexpr uint32_t kBOffset = kStages * kABytes;
  static constexpr uint32_t kSfaOffset = kBOffset + kStages * kBBytes;
  static constexpr uint32_t kSfbOffset = kSfaOffset + kStages * kSfaBytes;
  static constexpr uint32_t kBarrierOffset = kSfbOffset + kStages * kSfbBytes;
  static constexpr uint32_t kBarriers = 2 * kStages + 2 * kAccStages;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  // Tile starts of up to kSharedGroups groups, copied once per CTA: the per-tile binary search
  // then runs on shared memory instead of on a chain of dependent L2 round trips (measured:
  // with the search in global memory the tensor pipe was busy 24 % of a launch).
  static constexpr uint32_t kSharedGroups = 1024;
  static constexpr uint32_t kStartsOffset = kMiscOffset + 16;
  static constexpr uint32_t kDynamicBytes = kStartsOffset + (kSharedGroups + 1) * 4 + 1024;
  // Tensor memory: the accumulators, then per stage 16 columns of A scales and 16 per 128 rows
  // of B scales ([K atom][128-row tile of B][4 columns], the order the MMA reads them in).
  static constexpr uint32_t kSfColumn = kAccStages * BN;
  static constexpr uint32_t kSfColumnsPerStage = 4 * kAtomsK * (1 + kAtomsN);
  static_assert(kSfColumn + kStages * kSfColumnsPerStage <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

// One routed group, written by the set-up kernel.
struct alignas(32) Group {
  uint32_t matrix;
  uint32_t rows;         // 0 for a skipped group
  uint32_t a_row;        // first row in A
  uint32_t c_row;        // first row in C
  uint32_t scale_tile;   // first 128-row tile of the group's A scales
  uint32_t tile_start;   // tiles in groups before this one
  uint32_t padding[2];
};

struct Side {
  CUtensorMap a[kPieceMaps];   // box rows 128 >> index
  CUtensorMap b;               // [matrices, N, K/2], box 128 B x 128 rows x 1
  const uint8_t* a_scales;
  const uint8_t* b_scales;
  const float* alphas;
  __nv_bfloat16* c;
  // Fused SwiGLU + NVFP4 requantisation (null `codes`: plain bf16 output). The matrices then
  // hold gate and up rows interleaved in runs of 16 (rows 32 b .. 32 b + 15 = gate rows
  // 16 b .. 16 b + 15, rows 32 b + 16 .. 32 b + 31 = the up rows of the same columns), so that
  // one 32-column piece of an accumulator row is one 16-element block of the activation.
  uint2* codes;               // [capacity, n / 4] bytes: E2M1 codes of silu(gate) * up
  uint8_t* out_scales;        // swizzled UE4M3 scales of that tensor, rows as in C
  const float* out_global;    // its tensor scale (device)
};

struct Sides {
  Side side[2];
};

// Exclusive scan of per-group tile counts over one 1024-thread block (serial carry across
// chunks). `count_of(group)` returns the group's record with `tile_start` still unset.
template <typename Describe>
__device__ __forceinline__ void scan_groups(uint32_t groups, uint32_t tiles_n, Group* records,
                                            uint32_t* total_tiles, Describe describe) {
  __shared__ uint32_t warp_totals[32];
  __shared__ uint32_t carry;
  if (threadIdx.x == 0) carry = 0u;
  __syncthreads();
  for (uint32_t base = 0; base < groups; base += 1024u) {
    const uint32_t group = base + threadIdx.x;
    Group record = {};
    uint32_t count = 0u;
    if (group < groups) {
      record = describe(group);
      count = ((record.rows + kBlockM - 1u) / kBlockM) * tiles_n;
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
    if (group < groups) {
      record.tile_start = exclusive;
      records[group] = record;
    }
    __syncthreads();
    if (threadIdx.x == 1023u) carry = exclusive + count;
    __syncthreads();
  }
  if (threadIdx.x == 0) *total_tiles = carry;
}

__global__ void __launch_bounds__(1024)
grouped_fp4_variable_setup_kernel(const unsigned int* __restrict__ indices,
                                  const unsigned int* __restrict__ rows,
                                  const unsigned int* __restrict__ offsets,
                                  const unsigned int* __restrict__ scale_offsets, uint32_t groups,
                                  uint32_t matrices, uint32_t max_rows, uint32_t tiles_n,
                                  Group* __restrict__ records, uint32_t* __restrict__ total_tiles) {
  // The routing arrays come from the kernel before this one; the main kernel after this one may
  // set itself up meanwhile.
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  scan_groups(groups, tiles_n, records, total_tiles, [&](uint32_t group) {
    Group record = {};
    record.matrix = indices[group];
    record.rows = record.matrix < matrices ? min(rows[group], max_rows) : 0u;
    record.a_row = offsets[group];
    record.c_row = offsets[group];
    record.scale_tile = scale_offsets[group] / 128u;
    return record;
  });
}

__global__ void __launch_bounds__(1024)
grouped_fp4_indexed_setup_kernel(const unsigned int* __restrict__ selected, uint32_t groups,
                                 uint32_t matrices, uint32_t m, bool broadcast_input,
                                 uint32_t tiles_n, Group* __restrict__ records,
                                 uint32_t* __restrict__ total_tiles) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  scan_groups(groups, tiles_n, records, total_tiles, [&](uint32_t group) {
    const uint32_t input_group = broadcast_input ? 0u : group;
    Group record = {};
    record.matrix = selected[group];
    record.rows = record.matrix < matrices ? m : 0u;
    record.a_row = input_group * m;
    record.c_row = group * m;
    record.scale_tile = input_group * ((m + 127u) / 128u);
    return record;
  });
}

struct Tile {
  Group group;
  uint32_t row_tile;
  uint32_t valid_rows;  // 1..128
  uint32_t n0;
};

// Linear tile index (within one side) -> tile. Inside a group, row tiles vary fastest.
__device__ __forceinline__ Tile locate(uint32_t index, const Group* __restrict__ records,
                                       uint32_t groups, const uint32_t* shared_starts,
                                       uint32_t block_n) {
  uint32_t low = 0u, high = groups;       // last group whose start is <= index
  if (shared_starts != nullptr) {
    while (high - low > 1u) {
      const uint32_t middle = (low + high) / 2u;
      if (shared_starts[middle] <= index) low = middle; else high = middle;
    }
    // Groups without tiles share their start with the next group; step past them.
    while (low + 1u < groups && shared_starts[low + 1u] <= index) ++low;
  } else {
    while (high - low > 1u) {
      const uint32_t middle = (low + high) / 2u;
      if (__ldg(&records[middle].tile_start) <= index) low = middle; else high = middle;
    }
    while (low + 1u < groups && __ldg(&records[low + 1u].tile_start) <= index) ++low;
  }
  Tile tile;
  const uint4 first = __ldg(reinterpret_cast<const uint4*>(records + low));
  const uint4 second = __ldg(reinterpret_cast<const uint4*>(records + low) + 1);
  tile.group.matrix = first.x;
  tile.group.rows = first.y;
  tile.group.a_row = first.z;
  tile.group.c_row = first.w;
  tile.group.scale_tile = second.x;
  tile.group.tile_start = second.y;
  const uint32_t row_tiles = (tile.group.rows + kBlockM - 1u) / kBlockM;
  const uint32_t local = index - tile.group.tile_start;
  tile.row_tile = local % row_tiles;
  tile.valid_rows = min(kBlockM, tile.group.rows - tile.row_tile * kBlockM);
  tile.n0 = (local / row_tiles) * block_n;
  return tile;
}

template <uint32_t BN, uint32_t SETS>
__global__ void __launch_bounds__(threads_for(SETS), 1)
grouped_fp4_kernel(const __grid_constant__ Sides sides, uint32_t side_count,
                   const Group* __restrict__ records, const uint32_t* __restrict__ total_tiles,
                   uint32_t groups, uint32_t n, uint32_t k, uint32_t* __restrict__ status) {
  using L = Layout<BN>;
  constexpr uint32_t kStages = L::kStages;
  constexpr uint32_t kAccStages = L::kAccStages;
  constexpr uint32_t kThreads = threads_for(SETS);
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_a = shared;
  uint8_t* shared_b = shared + L::kBOffset;
  uint8_t* shared_sfa = shared + L::kSfaOffset;
  uint8_t* shared_sfb = shared + L::kSfbOffset;
  uint64_t* full = reinterpret_cast<uint64_t*>(shared + L::kBarrierOffset);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;
  uint64_t* acc_empty = acc_full + kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(shared + L::kMiscOffset);
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const uint32_t warp = threadIdx.x / 32u;
  const uint32_t lane = threadIdx.x % 32u;

  if (threadIdx.x == 0) {
    for (uint32_t stage = 0; stage < kStages; ++stage) {
      ptx::mbarrier_init(&full[stage], 1);
      ptx::mbarrier_init(&empty[stage], 1);
    }
    for (uint32_t stage = 0; stage < kAccStages; ++stage) {
      ptx::mbarrier_init(&acc_full[stage], 1);
      ptx::mbarrier_init(&acc_empty[stage], 4u * SETS);
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&sides.side[0].a[0]);
    ptx::prefetch_tensor_map(&sides.side[0].b);
  }
  if (warp == 1) {
    ptx::tmem_allocate(tmem_slot, kTmemColumns);
    ptx::tmem_relinquish();
  }
  // Barriers, tensor memory and the tensor-map prefetch above needed nothing from global memory
  // and may have run beside the set-up kernel; its records are read from here on.
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  uint32_t* starts_table = reinterpret_cast<uint32_t*>(shared + L::kStartsOffset);
  const uint32_t* shared_starts = groups <= L::kSharedGroups ? starts_table : nullptr;
  if (shared_starts != nullptr) {
    for (uint32_t group = threadIdx.x; group < groups; group += kThreads) {
      starts_table[group] = __ldg(&records[group].tile_start);
    }
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t side_tiles = __ldg(total_tiles);
  const uint32_t tiles = side_tiles * side_count;
  const uint32_t atoms_k = k / 64u;
  const uint32_t atoms_n = (n + 127u) / 128u;
  const uint32_t k_stages = (k + kStageElements - 1u) / kStageElements;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool running = true;
      // The next tile's record is fetched while this tile's loads are being issued.
      Tile upcoming = {};
      if (blockIdx.x < tiles) {
        upcoming = locate(blockIdx.x >= side_tiles ? blockIdx.x - side_tiles : blockIdx.x, records,
                          groups, shared_starts, BN);
      }
      for (uint32_t index = blockIdx.x; running && index < tiles; index += gridDim.x) {
        const Side& side = sides.side[index >= side_tiles ? 1 : 0];
        const Tile tile = upcoming;
        const uint32_t following = index + gridDim.x;
        if (following < tiles) {
          upcoming = locate(following >= side_tiles ? following - side_tiles : following, records,
                            groups, shared_starts, BN);
        }
        const uint32_t a_row = tile.group.a_row + tile.row_tile * kBlockM;
        const uint8_t* a_scales =
            side.a_scales + static_cast<size_t>(tile.group.scale_tile + tile.row_tile) * atoms_k * kAtomBytes;
        const uint8_t* b_scales =
            side.b_scales + (static_cast<size_t>(tile.group.matrix) * atoms_n + tile.n0 / 128u) *
                                atoms_k * kAtomBytes;
        for (uint32_t ks = 0; ks < k_stages; ++ks) {
          if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          const uint32_t atoms_here = min(kAtomsK, atoms_k - ks * kAtomsK);
          ptx::mbarrier_arrive_expect_tx(
              &full[stage],
              tile.valid_rows * kStageBytesK + L::kBBytes + (1u + L::kAtomsN) * atoms_here * kAtomBytes);
          uint8_t* a_stage = shared_a + stage * L::kABytes;
          const int32_t x = static_cast<int32_t>(ks * kStageBytesK);
          if (tile.valid_rows == kBlockM) {
            ptx::tma_load_2d(a_stage, &side.a[0], &full[stage], x, static_cast<int32_t>(a_row));
          } else {
            // Ragged last tile of a group: pieces of 64, 32, ... 1 rows. A piece of p rows
            // starts at a multiple of p rows, so pieces of 8 or more rows start on the
            // 1024-byte swizzle period and smaller ones keep their place inside it.
            uint32_t done = 0u;
#pragma unroll
            for (uint32_t piece = 1; piece < kPieceMaps; ++piece) {
              const uint32_t piece_rows = kBlockM >> piece;
              if ((tile.valid_rows & piece_rows) != 0u) {
                ptx::tma_load_2d(a_stage + done * kStageBytesK, &side.a[piece], &full[stage], x,
                                 static_cast<int32_t>(a_row + done));
                done += piece_rows;
              }
            }
          }
          ptx::tma_load_3d(shared_b + stage * L::kBBytes, &side.b, &full[stage], x,
                           static_cast<int32_t>(tile.n0), static_cast<int32_t>(tile.group.matrix));
          ptx::bulk_load(shared_sfa + stage * L::kSfaBytes,
                         a_scales + static_cast<size_t>(ks) * kAtomsK * kAtomBytes,
                         atoms_here * kAtomBytes, &full[stage]);
#pragma unroll
          for (uint32_t tile_n = 0; tile_n < L::kAtomsN; ++tile_n) {     // 128-row scale tiles of B
            ptx::bulk_load(shared_sfb + stage * L::kSfbBytes + tile_n * kAtomsK * kAtomBytes,
                           b_scales + (static_cast<size_t>(tile_n) * atoms_k + static_cast<size_t>(ks) * kAtomsK) * kAtomBytes,
                           atoms_here * kAtomBytes, &full[stage]);
          }
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
    // -------------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::make_block_scaled_idesc(
          ptx::kFormatE2M1_mxf4, ptx::kFormatE2M1_mxf4, kBlockM, BN, false);
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      for (uint32_t index = blockIdx.x; running && index < tiles; index += gridDim.x) {
        if (!ptx::mbarrier_wait(&acc_empty[acc_stage], acc_phase ^ 1u, abort)) break;
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * BN;
        for (uint32_t ks = 0; ks < k_stages; ++ks) {
          if (!ptx::mbarrier_wait(&full[stage], phase, abort)) {
            running = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t atoms_here = min(kAtomsK, atoms_k - ks * kAtomsK);
          const uint32_t sfa_tmem = tmem_base + L::kSfColumn + stage * L::kSfColumnsPerStage;
          const uint32_t sfb_tmem = sfa_tmem + 4u * kAtomsK;
          for (uint32_t atom = 0; atom < atoms_here; ++atom) {
            ptx::tcgen05_copy_scales(
                sfa_tmem + 4u * atom,
                ptx::make_scale_descriptor(
                    ptx::smem_address(shared_sfa + stage * L::kSfaBytes + atom * kAtomBytes)));
#pragma unroll
            for (uint32_t tile_n = 0; tile_n < L::kAtomsN; ++tile_n) {
              ptx::tcgen05_copy_scales(
                  sfb_tmem + 4u * (atom * L::kAtomsN + tile_n),
                  ptx::make_scale_descriptor(ptx::smem_address(
                      shared_sfb + stage * L::kSfbBytes + (tile_n * kAtomsK + atom) * kAtomBytes)));
            }
          }
          const uint64_t a_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_a + stage * L::kABytes));
          const uint64_t b_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_b + stage * L::kBBytes));
          for (uint32_t kb = 0; kb < atoms_here; ++kb) {
            // 32 bytes (64 codes) further along K inside the 128-byte swizzle span.
            ptx::mma_nvf4_block16(d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc,
                                  sfa_tmem + 4u * kb, sfb_tmem + 4u * kb * L::kAtomsN, (ks | kb) != 0u);
          }
          ptx::tcgen05_commit(&empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
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
  } else {
    // ---------------------------------------------------------------------- epilogue
    const uint32_t quarter = warp % 4u;
    const uint32_t set = (warp - 2u) / 4u;          // which share of the tile's columns
    const bool vector_stores = (n % 8u) == 0u;
    uint32_t acc_stage = 0, acc_phase = 0;
    // 32-byte stores need rows that start on 32-byte boundaries (n % 16 == 0 and such a base)
    const bool wide_stores = (n % 16u) == 0u &&
                             ((reinterpret_cast<uintptr_t>(sides.side[0].c) | reinterpret_cast<uintptr_t>(sides.side[1].c)) & 31u) == 0u;
    // The next tile's record and alpha are fetched while this tile is drained (two dependent
    // global loads after a search: about a microsecond if taken when the tile is due).
    Tile upcoming = {};
    float upcoming_alpha = 0.0f;
    if (blockIdx.x < tiles) {
      upcoming = locate(blockIdx.x >= side_tiles ? blockIdx.x - side_tiles : blockIdx.x, records, groups,
                        shared_starts, BN);
      upcoming_alpha = __ldg(sides.side[blockIdx.x >= side_tiles ? 1 : 0].alphas + upcoming.group.matrix);
    }
    for (uint32_t index = blockIdx.x; index < tiles; index += gridDim.x) {
      const Side& side = sides.side[index >= side_tiles ? 1 : 0];
      const Tile tile = upcoming;
      const float alpha = upcoming_alpha;
      if (!ptx::mbarrier_wait(&acc_full[acc_stage], acc_phase, abort)) break;
      ptx::tcgen05_fence_after();
      const uint32_t row_in_tile = quarter * 32u + lane;
      const uint32_t tmem_row = tmem_base + ((quarter * 32u) << 16) + acc_stage * BN;
      const bool row_valid = row_in_tile < tile.valid_rows;
      const uint32_t out_row = tile.group.c_row + tile.row_tile * kBlockM + row_in_tile;
      __nv_bfloat16* c_row = side.c + static_cast<size_t>(out_row) * n;

      // One 32-column piece of this thread's accumulator row.
      auto write_piece = [&](const uint32_t (&values)[32], uint32_t chunk) {
        const uint32_t column = tile.n0 + chunk * 32u;
        if (side.codes != nullptr) {
          // gate_up -> SwiGLU -> NVFP4: columns 0..15 of the piece are gate, 16..31 up, of output
          // block column / 32; each value is rounded to bf16 first, as the unfused path stores it.
          if (row_valid && column + 32u <= n) {
            uint32_t gate[8], up[8];
#pragma unroll
            for (uint32_t pair = 0; pair < 8u; ++pair) {
              const __nv_bfloat162 g = __floats2bfloat162_rn(__uint_as_float(values[2u * pair]) * alpha,
                                                             __uint_as_float(values[2u * pair + 1u]) * alpha);
              const __nv_bfloat162 u = __floats2bfloat162_rn(__uint_as_float(values[16u + 2u * pair]) * alpha,
                                                             __uint_as_float(values[17u + 2u * pair]) * alpha);
              gate[pair] = *reinterpret_cast<const uint32_t*>(&g);
              up[pair] = *reinterpret_cast<const uint32_t*>(&u);
            }
            const uint4 first = nvfp4_block::swiglu8(make_uint4(gate[0], gate[1], gate[2], gate[3]),
                                                     make_uint4(up[0], up[1], up[2], up[3]));
            const uint4 second = nvfp4_block::swiglu8(make_uint4(gate[4], gate[5], gate[6], gate[7]),
                                                      make_uint4(up[4], up[5], up[6], up[7]));
            uint8_t scale_code = 0u;
            const uint2 packed = nvfp4_block::quantize_block16(first, second, __ldg(side.out_global), &scale_code);
            const uint32_t blocks = n / 32u;
            side.codes[static_cast<size_t>(out_row) * blocks + column / 32u] = packed;
            side.out_scales[scale_offset(out_row, column / 32u, blocks)] = scale_code;
          }
        } else if (row_valid && column < n) {
          __nv_bfloat16* destination = c_row + column;
          if (vector_stores && column + 32u <= n) {
            uint32_t packed[16];
#pragma unroll
            for (uint32_t pair = 0; pair < 16u; ++pair) {
              const __nv_bfloat162 two = __floats2bfloat162_rn(__uint_as_float(values[pair * 2u]) * alpha,
                                                             __uint_as_float(values[pair * 2u + 1u]) * alpha);
              packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
            }
            if (wide_stores) {
              // 32 bytes per store: every store fills whole 32-byte sectors. With 16-byte stores
              // the same rows cost twice the L1 -> L2 write traffic (measured: 265 MB for a 134 MB
              // output), which this kernel's L2-bound launches cannot spare.
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
                destination[item] = __float2bfloat16_rn(__uint_as_float(values[item]) * alpha);
              }
            }
          }
        }
      };

      // Pieces alternate between two register buffers: the tensor-memory load of the next piece
      // is in flight while this one is converted and stored. The accumulator goes back to the
      // MMA warp as soon as its last piece has been read.
      constexpr uint32_t kSetPieces = BN / 32u / SETS;
      const uint32_t first_piece = set * kSetPieces, kPieces = first_piece + kSetPieces;
      uint32_t even[32], odd[32];
      ptx::tmem_load_32x32(tmem_row + first_piece * 32u, even);
      ptx::tmem_load_wait();
#pragma unroll 1
      for (uint32_t chunk = first_piece; chunk < kPieces; chunk += 2u) {
        ptx::tmem_load_32x32(tmem_row + (chunk + 1u) * 32u, odd);
        if (chunk == first_piece) {
          // first use of the wait: fetch the next tile's record behind the loads already issued
          const uint32_t following = index + gridDim.x;
          if (following < tiles) {
            upcoming = locate(following >= side_tiles ? following - side_tiles : following, records, groups,
                              shared_starts, BN);
            upcoming_alpha = __ldg(sides.side[following >= side_tiles ? 1 : 0].alphas + upcoming.group.matrix);
          }
        }
        write_piece(even, chunk);
        ptx::tmem_load_wait();
        if (chunk + 2u < kPieces) {
          ptx::tmem_load_32x32(tmem_row + (chunk + 2u) * 32u, even);
        } else {
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbarrier_arrive(&acc_empty[acc_stage]);
        }
        write_piece(odd, chunk + 1u);
        ptx::tmem_load_wait();
      }
      if (++acc_stage == kAccStages) {
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

enum class Mode { kVariable, kPaired, kIndexed };

using Kernel = void (*)(const Sides, uint32_t, const Group*, const uint32_t*, uint32_t, uint32_t, uint32_t,
                        uint32_t*);

inline Kernel kernel_for(bool wide, uint32_t epilogue_sets) {
  if (wide) return epilogue_sets == 2u ? grouped_fp4_kernel<256, 2> : grouped_fp4_kernel<256, 1>;
  return epilogue_sets == 2u ? grouped_fp4_kernel<128, 2> : grouped_fp4_kernel<128, 1>;
}

struct Plan {
  Mode mode;
  int groups, matrices, max_rows, n, k;
  bool broadcast_input;
  int device, sm_count;
  cudaStream_t stream;
  Group* records;            // device, one per group
  uint32_t* total_tiles;     // device
  uint32_t* status;          // pinned
  const void* cached_a[2];
  const void* cached_b[2];
  uint32_t block_n;          // tile width: 256 when n is a multiple of it, else 128
  uint32_t epilogue_sets;    // sets of four epilogue warps: 1 or 2, 0 = chosen per launch
  Sides sides;
};

int encode_weight_map(CUtensorMap* map, const void* base, uint64_t matrices, uint64_t n,
                      uint64_t k_bytes, uint32_t block_n) {
  EncodeTiled encode = encode_tiled_entry();
  if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dimensions[3] = {k_bytes, n, matrices};
  const cuuint64_t strides[2] = {k_bytes, n * k_bytes};
  const cuuint32_t box[3] = {kStageBytesK, block_n, 1u};
  const cuuint32_t element_strides[3] = {1u, 1u, 1u};
  return static_cast<int>(encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3u, const_cast<void*>(base),
                                 dimensions, strides, box, element_strides,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
}

int create(Mode mode, int groups, int matrices, int max_rows, int n, int k, bool broadcast_input,
           void* stream, void** output) {
  if (groups <= 0 || matrices <= 0 || max_rows <= 0 || n <= 0 || k <= 0 || k % 64 != 0 ||
      stream == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->mode = mode;
  plan->groups = groups;
  plan->matrices = matrices;
  plan->max_rows = max_rows;
  plan->n = n;
  plan->k = k;
  plan->broadcast_input = broadcast_input;
  plan->stream = static_cast<cudaStream_t>(stream);
  int status = static_cast<int>(cudaGetDevice(&plan->device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&plan->sm_count,
                                                     cudaDevAttrMultiProcessorCount, plan->device));
  }
  if (status == 0) {
    status = static_cast<int>(cudaMallocAsync(reinterpret_cast<void**>(&plan->records),
                                              static_cast<size_t>(groups) * sizeof(Group),
                                              plan->stream));
  }
  if (status == 0) {
    status = static_cast<int>(cudaMallocAsync(reinterpret_cast<void**>(&plan->total_tiles),
                                              sizeof(uint32_t), plan->stream));
  }
  if (status == 0) {
    status = static_cast<int>(cudaHostAlloc(reinterpret_cast<void**>(&plan->status),
                                            sizeof(uint32_t), cudaHostAllocMapped));
  }
  for (uint32_t variant = 0; variant < 4u && status == 0; ++variant) {
    status = static_cast<int>(cudaFuncSetAttribute(kernel_for(variant / 2u != 0u, variant % 2u + 1u),
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   variant / 2u != 0u ? Layout<256>::kDynamicBytes
                                                                      : Layout<128>::kDynamicBytes));
  }
  // 128-wide tiles by default. MIRCUDA_B200_GROUPED_FP4_BN=256 selects the wide ones where they
  // tile N exactly: measured at the Qwen3-30B-A3B shapes they lose (gate_up with the fused
  // epilogue 0.138 against 0.111 ms, down equal), because with one accumulator the epilogue no
  // longer overlaps the next tile's MMAs and the epilogue, not the operand stream, is what a
  // tile of these K extents waits for.
  plan->block_n = 128u;
  if (const char* forced = std::getenv("MIRCUDA_B200_GROUPED_FP4_BN")) {
    if (std::atoi(forced) == 256 && n % 256 == 0) plan->block_n = 256u;
  }
  // Epilogue warps: chosen per launch (see run()); MIRCUDA_B200_GROUPED_FP4_EPILOGUE=4 or 8 forces one or two sets.
  plan->epilogue_sets = 0u;
  if (const char* forced = std::getenv("MIRCUDA_B200_GROUPED_FP4_EPILOGUE")) {
    if (std::atoi(forced) == 8) plan->epilogue_sets = 2u;
    if (std::atoi(forced) == 4) plan->epilogue_sets = 1u;
  }
  if (status != 0) {
    if (plan->records != nullptr) cudaFreeAsync(plan->records, plan->stream);
    if (plan->total_tiles != nullptr) cudaFreeAsync(plan->total_tiles, plan->stream);
    if (plan->status != nullptr) cudaFreeHost(plan->status);
    delete plan;
    return status;
  }
  *plan->status = 0u;
  *output = plan;
  return 0;
}

void destroy(void* raw) {
  auto* plan = static_cast<Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->records != nullptr) cudaFreeAsync(plan->records, plan->stream);
  if (plan->total_tiles != nullptr) cudaFreeAsync(plan->total_tiles, plan->stream);
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}

struct Operands {
  const void* a;
  const void* a_scales;
  const void* b;
  const void* b_scales;
  const void* alphas;
  void* c;                    // bf16 output, or the code bytes when `out_scales` is given
  void* out_scales = nullptr;
  const void* out_global = nullptr;
};

int bind_side(Plan* plan, int index, const Operands& operands) {
  if (operands.a == nullptr || operands.a_scales == nullptr || operands.b == nullptr ||
      operands.b_scales == nullptr || operands.alphas == nullptr || operands.c == nullptr) {
    return -1;
  }
  if (((reinterpret_cast<uintptr_t>(operands.a) | reinterpret_cast<uintptr_t>(operands.a_scales) |
        reinterpret_cast<uintptr_t>(operands.b) | reinterpret_cast<uintptr_t>(operands.b_scales) |
        reinterpret_cast<uintptr_t>(operands.c)) & 15u) != 0u) {
    return -1;
  }
  Side& side = plan->sides.side[index];
  const uint64_t k_bytes = static_cast<uint64_t>(plan->k) / 2u;
  if (operands.a != plan->cached_a[index]) {
    // The row extent of the compact matrix is not part of these interfaces; loads are issued
    // only for rows a group owns, so the map's row bound is left wide open.
    for (uint32_t piece = 0; piece < kPieceMaps; ++piece) {
      const int status = encode_k_major_map(&side.a[piece], operands.a, 0x7fffffffull, k_bytes, 1u,
                                            kBlockM >> piece);
      if (status != 0) return status;
    }
    plan->cached_a[index] = operands.a;
  }
  if (operands.b != plan->cached_b[index]) {
    const int status = encode_weight_map(&side.b, operands.b, plan->matrices, plan->n, k_bytes, plan->block_n);
    if (status != 0) return status;
    plan->cached_b[index] = operands.b;
  }
  side.a_scales = static_cast<const uint8_t*>(operands.a_scales);
  side.b_scales = static_cast<const uint8_t*>(operands.b_scales);
  side.alphas = static_cast<const float*>(operands.alphas);
  if (operands.out_scales != nullptr) {
    if (operands.out_global == nullptr || plan->n % 32 != 0) return -1;
    side.c = nullptr;
    side.codes = static_cast<uint2*>(operands.c);
    side.out_scales = static_cast<uint8_t*>(operands.out_scales);
    side.out_global = static_cast<const float*>(operands.out_global);
  } else {
    side.c = static_cast<__nv_bfloat16*>(operands.c);
    side.codes = nullptr;
    side.out_scales = nullptr;
    side.out_global = nullptr;
  }
  return 0;
}

int run(Plan* plan, uint32_t side_count) {
  const bool wide = plan->block_n == 256u;
  // Two sets of epilogue warps where the epilogue also does SwiGLU and the requantisation
  // (measured: gate_up 0.116 -> 0.112 ms); one set for plain bf16 outputs, where eight warps
  // storing at once were slower (down 0.081 -> 0.086 ms).
  const uint32_t sets = plan->epilogue_sets != 0u ? plan->epilogue_sets
                                                  : (plan->sides.side[0].codes != nullptr ? 2u : 1u);
  return launch_after_dependency(kernel_for(wide, sets), dim3(plan->sm_count), dim3(threads_for(sets)),
                                 wide ? Layout<256>::kDynamicBytes : Layout<128>::kDynamicBytes, plan->stream,
                                 plan->sides, side_count, plan->records, plan->total_tiles,
                                 static_cast<uint32_t>(plan->groups), static_cast<uint32_t>(plan->n),
                                 static_cast<uint32_t>(plan->k), plan->status);
}

int check(void* raw, void* stream, Mode mode, Plan** plan) {
  if (raw == nullptr || stream == nullptr) return -1;
  *plan = static_cast<Plan*>(raw);
  if ((*plan)->mode != mode) return -1;
  if (static_cast<cudaStream_t>(stream) != (*plan)->stream) return -1;
  if (*static_cast<volatile uint32_t*>((*plan)->status) != 0u) return -3;
  return 0;
}

int setup_variable(Plan* plan, const unsigned int* indices, const unsigned int* rows,
                   const unsigned int* offsets, const unsigned int* scale_offsets) {
  if (indices == nullptr || rows == nullptr || offsets == nullptr || scale_offsets == nullptr) {
    return -1;
  }
  const uint32_t tiles_n = (plan->n + plan->block_n - 1u) / plan->block_n;
  return launch_after_dependency(grouped_fp4_variable_setup_kernel, dim3(1), dim3(1024), 0, plan->stream, indices,
                                 rows, offsets, scale_offsets, static_cast<uint32_t>(plan->groups),
                                 static_cast<uint32_t>(plan->matrices), static_cast<uint32_t>(plan->max_rows),
                                 tiles_n, plan->records, plan->total_tiles);
}

}  // namespace grouped_fp4
}  // namespace mircuda_b200

using mircuda_b200::grouped_fp4::Mode;
using mircuda_b200::grouped_fp4::Operands;
using mircuda_b200::grouped_fp4::Plan;

extern "C" int mircuda_variable_grouped_fp4_create(int groups, int matrices, int max_m, int n,
                                                   int k, void* stream, void** output) {
  return mircuda_b200::grouped_fp4::create(Mode::kVariable, groups, matrices, max_m, n, k, false,
                                           stream, output);
}

extern "C" int mircuda_variable_grouped_fp4_execute(
    void* raw, void* stream, const void* a, const void* a_scales, const void* b,
    const void* b_scales, const void* alphas, const unsigned int* indices,
    const unsigned int* rows, const unsigned int* offsets, const unsigned int* scale_offsets,
    void* c) {
  using namespace mircuda_b200::grouped_fp4;
  Plan* plan = nullptr;
  int status = check(raw, stream, Mode::kVariable, &plan);
  if (status == 0) status = bind_side(plan, 0, Operands{a, a_scales, b, b_scales, alphas, c});
  if (status == 0) status = setup_variable(plan, indices, rows, offsets, scale_offsets);
  if (status == 0) status = run(plan, 1u);
  return status;
}

extern "C" int mircuda_b200_variable_grouped_fp4_execute_swiglu(
    void* raw, void* stream, const void* a, const void* a_scales, const void* b,
    const void* b_scales, const void* alphas, const unsigned int* indices,
    const unsigned int* rows, const unsigned int* offsets, const unsigned int* scale_offsets,
    const void* global_scale, void* codes, void* scales) {
  using namespace mircuda_b200::grouped_fp4;
  Plan* plan = nullptr;
  int status = check(raw, stream, Mode::kVariable, &plan);
  if (status == 0 && (global_scale == nullptr || scales == nullptr)) status = -1;
  if (status == 0) {
    status = bind_side(plan, 0, Operands{a, a_scales, b, b_scales, alphas, codes, scales, global_scale});
  }
  if (status == 0) status = setup_variable(plan, indices, rows, offsets, scale_offsets);
  if (status == 0) status = run(plan, 1u);
  return status;
}

extern "C" void mircuda_variable_grouped_fp4_destroy(void* raw) {
  mircuda_b200::grouped_fp4::destroy(raw);
}

extern "C" int mircuda_paired_variable_grouped_fp4_create(int groups, int matrices, int max_m,
                                                          int n, int k, void* stream,
                                                          void** output) {
  return mircuda_b200::grouped_fp4::create(Mode::kPaired, groups, matrices, max_m, n, k, false,
                                           stream, output);
}

extern "C" int mircuda_paired_variable_grouped_fp4_execute(
    void* raw, void* stream, const void* left_a, const void* left_a_scales, const void* left_b,
    const void* left_b_scales, const void* left_alphas, const void* right_a,
    const void* right_a_scales, const void* right_b, const void* right_b_scales,
    const void* right_alphas, const unsigned int* indices, const unsigned int* rows,
    const unsigned int* offsets, const unsigned int* scale_offsets, void* left_c, void* right_c) {
  using namespace mircuda_b200::grouped_fp4;
  Plan* plan = nullptr;
  int status = check(raw, stream, Mode::kPaired, &plan);
  if (status == 0) {
    status = bind_side(plan, 0, Operands{left_a, left_a_scales, left_b, left_b_scales, left_alphas, left_c});
  }
  if (status == 0) {
    status = bind_side(plan, 1,
                       Operands{right_a, right_a_scales, right_b, right_b_scales, right_alphas, right_c});
  }
  if (status == 0) status = setup_variable(plan, indices, rows, offsets, scale_offsets);
  if (status == 0) status = run(plan, 2u);
  return status;
}

extern "C" void mircuda_paired_variable_grouped_fp4_destroy(void* raw) {
  mircuda_b200::grouped_fp4::destroy(raw);
}

extern "C" int mircuda_grouped_fp4_create(int groups, int experts, int m, int n, int k,
                                          bool broadcast_input, void* stream, void** output) {
  return mircuda_b200::grouped_fp4::create(Mode::kIndexed, groups, experts, m, n, k,
                                           broadcast_input, stream, output);
}

extern "C" int mircuda_grouped_fp4_execute(void* raw, void* stream, const void* a,
                                           const void* a_scales, const void* b,
                                           const void* b_scales, const void* alphas,
                                           const unsigned int* selected, void* c) {
  using namespace mircuda_b200::grouped_fp4;
  Plan* plan = nullptr;
  int status = check(raw, stream, Mode::kIndexed, &plan);
  if (status == 0) status = bind_side(plan, 0, Operands{a, a_scales, b, b_scales, alphas, c});
  if (status == 0 && selected == nullptr) status = -1;
  if (status != 0) return status;
  const uint32_t tiles_n = (plan->n + plan->block_n - 1u) / plan->block_n;
  status = mircuda_b200::launch_after_dependency(grouped_fp4_indexed_setup_kernel, dim3(1), dim3(1024), 0, plan->stream,
                                   selected, static_cast<uint32_t>(plan->groups),
                                   static_cast<uint32_t>(plan->matrices), static_cast<uint32_t>(plan->max_rows),
                                   plan->broadcast_input, tiles_n, plan->records, plan->total_tiles);
  if (status == 0) status = run(plan, 1u);
  return status;
}

extern "C" void mircuda_grouped_fp4_destroy(void* raw) { mircuda_b200::grouped_fp4::destroy(raw); }
