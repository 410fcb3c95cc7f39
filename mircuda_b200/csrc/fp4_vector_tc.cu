// FP4 x FP4 GEMV (M = 1) on the tensor cores of sm_100a: the weights are the 128-row operand
// of tcgen05.mma.kind::mxf4nvf4.block_scale.block16 and the activation vector is row 0 of a
// 16-row second operand whose other rows are zero (TMA fills them: the tensor has one row).
// The tensor core decodes E2M1 and applies both UE4M3 block scales itself, so no thread
// touches a weight: bytes go HBM -> shared memory (TMA) -> tensor core, and the kernel is
// bound by how many bytes it keeps in flight, not by arithmetic.
//
// One persistent 192-thread CTA per SM. The row tiles' K stages (256 elements each), laid end
// to end, are cut into one equal contiguous range per CTA, so every SM streams the same number
// of bytes whatever the shape, and the eight-stage ring (22 KB a stage: 16 KB of weights, their
// four scale atoms, the 2 KB activation box, its four atoms) never drains where a range crosses
// from one row tile into the next. Warp 0 issues the loads, warp 1 copies the scale atoms
// into tensor memory and issues four MMAs per stage, warps 2-5 read column 0 of the
// accumulator (four accumulator stages, so a slow hand-over does not hold the MMAs up). K
// parts of one row tile meet in a scratch array; the warp that arrives last for its 32 rows
// (a counter per quarter of a row tile, no spinning, no barrier between warps) adds them in a
// fixed order, applies alpha and writes bf16, which keeps results deterministic. Every
// mbarrier wait is bounded.
#include "fp4_vector_tc.hpp"

#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdint>
#include <new>

#include "ptx.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace fp4_vector_tc {

constexpr uint32_t kTileRows = 128;
constexpr uint32_t kVectorRows = 16;       // rows of the second operand; only row 0 exists
constexpr uint32_t kStageBytesK = 128;     // 256 E2M1 codes per stage row
constexpr uint32_t kStageElements = 256;
constexpr uint32_t kAtomBytes = 512;
constexpr uint32_t kAtomsK = 4;            // scale atoms (64 K-elements each) per stage
constexpr uint32_t kThreads = 192;
constexpr uint32_t kStages = 8;
constexpr uint32_t kAccStages = 4;
constexpr uint32_t kAccColumns = 32;       // tensor-memory columns per accumulator stage
constexpr uint32_t kTmemColumns = 512;

struct Layout {
  static constexpr uint32_t kWeightBytes = kTileRows * kStageBytesK;          // 16 KB
  static constexpr uint32_t kVectorBytes = kVectorRows * kStageBytesK;        // 2 KB
  static constexpr uint32_t kSfBytes = kAtomsK * kAtomBytes;                  // 2 KB per operand
  static constexpr uint32_t kVectorOffset = kStages * kWeightBytes;
  static constexpr uint32_t kSfwOffset = kVectorOffset + kStages * kVectorBytes;
  static constexpr uint32_t kSfxOffset = kSfwOffset + kStages * kSfBytes;
  static constexpr uint32_t kBarrierOffset = kSfxOffset + kStages * kSfBytes;
  static constexpr uint32_t kBarriers = 2 * kStages + 2 * kAccStages;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  static constexpr uint32_t kDynamicBytes = kMiscOffset + 32 + 1024;
  static constexpr uint32_t kSfColumn = kAccStages * kAccColumns;
  static constexpr uint32_t kSfColumnsPerStage = 8 * kAtomsK;
  static_assert(kSfColumn + kStages * kSfColumnsPerStage <= kTmemColumns, "tensor memory budget");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

struct Plan {
  int n, k;
  uint32_t row_tiles, grid, max_contributors;
  int sm_count;
  cudaStream_t stream;
  float* partials;            // [max_contributors][row_tiles * 128]
  unsigned int* counters;     // [row_tiles][4], zero between launches
  uint32_t* status;           // pinned; set when a bounded wait ran out
  const void* cached_weight;
  const void* cached_input;
  CUtensorMap weight_map;     // [n, k/2] bytes, box 128 B x 128 rows, 128-byte swizzle
  CUtensorMap input_map;      // [1, k/2] bytes, box 128 B x 16 rows
};

__device__ __forceinline__ uint32_t tmem_load_column(uint32_t address) {
  uint32_t value;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(value) : "r"(address) : "memory");
  return value;
}

// The work is the row tiles' K stages laid end to end (row tile major); CTA b owns the
// stages [total * b / grid, total * (b + 1) / grid), so every CTA streams the same number of
// bytes (one stage more or less) whatever the shape. Its range is walked as segments, one per
// row tile it touches. A row tile cut over several CTAs has one contributor per CTA, numbered
// (`slot`) from the CTA that owns the tile's first stage.
struct Segment {
  uint32_t row_tile, first, last;     // stages [first, last) of the row tile
  uint32_t slot, contributors;
};

__host__ __device__ __forceinline__ uint32_t owner_of(uint64_t stage, uint64_t total, uint32_t grid) {
  return static_cast<uint32_t>(((stage + 1u) * grid - 1u) / total);
}

struct Walk {
  uint64_t position, end, total;
  uint32_t k_stages, grid, cta;

  __device__ __forceinline__ Walk(uint32_t row_tiles, uint32_t stages, uint32_t ctas, uint32_t index)
      : total(static_cast<uint64_t>(row_tiles) * stages), k_stages(stages), grid(ctas), cta(index) {
    position = total * index / ctas;
    end = total * (index + 1u) / ctas;
  }

  __device__ __forceinline__ bool next(Segment& segment) {
    if (position >= end) return false;
    segment.row_tile = static_cast<uint32_t>(position / k_stages);
    const uint64_t tile_begin = static_cast<uint64_t>(segment.row_tile) * k_stages;
    segment.first = static_cast<uint32_t>(position - tile_begin);
    const uint64_t stop = end < tile_begin + k_stages ? end : tile_begin + k_stages;
    segment.last = static_cast<uint32_t>(stop - tile_begin);
    const uint32_t first_owner = owner_of(tile_begin, total, grid);
    segment.slot = cta - first_owner;
    segment.contributors = owner_of(tile_begin + k_stages - 1u, total, grid) - first_owner + 1u;
    position = stop;
    return true;
  }
};

__global__ void __launch_bounds__(kThreads, 1)
fp4_vector_tc_kernel(const __grid_constant__ CUtensorMap weight_map,
                     const __grid_constant__ CUtensorMap input_map,
                     const uint8_t* __restrict__ weight_scales,
                     const uint8_t* __restrict__ input_scales, __nv_bfloat16* __restrict__ output,
                     float* __restrict__ partials, unsigned int* __restrict__ counters, uint32_t n,
                     uint32_t k, uint32_t row_tiles, float alpha, uint32_t* __restrict__ status) {
  using L = Layout;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_weight = shared;
  uint8_t* shared_vector = shared + L::kVectorOffset;
  uint8_t* shared_sfw = shared + L::kSfwOffset;
  uint8_t* shared_sfx = shared + L::kSfxOffset;
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
      ptx::mbarrier_init(&acc_empty[stage], 4);
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&weight_map);
    ptx::prefetch_tensor_map(&input_map);
  }
  if (warp == 1) {
    ptx::tmem_allocate(tmem_slot, kTmemColumns);
    ptx::tmem_relinquish();
  }
  // The loads do not need tensor memory: warp 0 only announces that the barriers exist and
  // starts streaming while warp 1 is still allocating; the other warps wait for both.
  uint32_t tmem_base = 0u;
  if (warp == 0) {
    __syncwarp();
    asm volatile("bar.arrive 2, 192;" ::: "memory");
  } else {
    ptx::tcgen05_fence_before();
    asm volatile("bar.sync 2, 192;" ::: "memory");
    ptx::tcgen05_fence_after();
    tmem_base = *tmem_slot;
  }

  const uint32_t atoms_k = k / 64u;
  const uint32_t k_stages = (k + kStageElements - 1u) / kStageElements;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool running = true;
      Walk walk(row_tiles, k_stages, gridDim.x, blockIdx.x);
      Segment segment;
      while (running && walk.next(segment)) {
        const uint32_t row_tile = segment.row_tile;
        const uint8_t* tile_scales = weight_scales + static_cast<size_t>(row_tile) * atoms_k * kAtomBytes;
        for (uint32_t ks = segment.first; ks < segment.last; ++ks) {
          if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          const uint32_t atoms_here = min(kAtomsK, atoms_k - ks * kAtomsK);
          ptx::mbarrier_arrive_expect_tx(
              &full[stage], L::kWeightBytes + L::kVectorBytes + 2u * atoms_here * kAtomBytes);
          const int32_t x = static_cast<int32_t>(ks * kStageBytesK);
          ptx::tma_load_2d(shared_weight + stage * L::kWeightBytes, &weight_map, &full[stage], x,
                           static_cast<int32_t>(row_tile * kTileRows));
          ptx::tma_load_2d(shared_vector + stage * L::kVectorBytes, &input_map, &full[stage], x, 0);
          ptx::bulk_load(shared_sfw + stage * L::kSfBytes,
                         tile_scales + static_cast<size_t>(ks) * kAtomsK * kAtomBytes,
                         atoms_here * kAtomBytes, &full[stage]);
          ptx::bulk_load(shared_sfx + stage * L::kSfBytes,
                         input_scales + static_cast<size_t>(ks) * kAtomsK * kAtomBytes,
                         atoms_here * kAtomBytes, &full[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort != 0u) {
        // Let copies already in flight land before the CTA's shared memory goes away.
        for (int spin = 0; spin < 256; ++spin) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::make_block_scaled_idesc(
          ptx::kFormatE2M1_mxf4, ptx::kFormatE2M1_mxf4, kTileRows, kVectorRows, false);
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0;
      bool running = true;
      Walk walk(row_tiles, k_stages, gridDim.x, blockIdx.x);
      Segment segment;
      while (running && walk.next(segment)) {
        const uint32_t first = segment.first, last = segment.last;
        if (!ptx::mbarrier_wait(&acc_empty[acc_stage], acc_phase ^ 1u, abort)) break;
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * kAccColumns;
        for (uint32_t ks = first; ks < last; ++ks) {
          if (!ptx::mbarrier_wait(&full[stage], phase, abort)) {
            running = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t atoms_here = min(kAtomsK, atoms_k - ks * kAtomsK);
          const uint32_t sfw_tmem = tmem_base + L::kSfColumn + stage * L::kSfColumnsPerStage;
          const uint32_t sfx_tmem = sfw_tmem + 4u * kAtomsK;
          for (uint32_t atom = 0; atom < atoms_here; ++atom) {
            ptx::tcgen05_copy_scales(
                sfw_tmem + 4u * atom,
                ptx::make_scale_descriptor(
                    ptx::smem_address(shared_sfw + stage * L::kSfBytes + atom * kAtomBytes)));
            ptx::tcgen05_copy_scales(
                sfx_tmem + 4u * atom,
                ptx::make_scale_descriptor(
                    ptx::smem_address(shared_sfx + stage * L::kSfBytes + atom * kAtomBytes)));
          }
          const uint64_t weight_descriptor = ptx::make_k_major_sw128_descriptor(
              ptx::smem_address(shared_weight + stage * L::kWeightBytes));
          const uint64_t vector_descriptor = ptx::make_k_major_sw128_descriptor(
              ptx::smem_address(shared_vector + stage * L::kVectorBytes));
          for (uint32_t kb = 0; kb < atoms_here; ++kb) {
            // 32 bytes (64 codes) further along K inside the 128-byte swizzle span.
            ptx::mma_nvf4_block16(d_tmem, weight_descriptor + 2u * kb, vector_descriptor + 2u * kb,
                                  idesc, sfw_tmem + 4u * kb, sfx_tmem + 4u * kb,
                                  (ks != first) || kb != 0u);
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
    const uint32_t row_in_tile = quarter * 32u + lane;
    const size_t padded_rows = static_cast<size_t>(row_tiles) * kTileRows;
    uint32_t acc_stage = 0, acc_phase = 0;
    Walk walk(row_tiles, k_stages, gridDim.x, blockIdx.x);
    Segment segment;
    while (walk.next(segment)) {
      const uint32_t row_tile = segment.row_tile;
      const uint32_t part = segment.slot, parts = segment.contributors;
      if (!__all_sync(0xffffffffu, ptx::mbarrier_wait(&acc_full[acc_stage], acc_phase, abort))) break;
      ptx::tcgen05_fence_after();
      const float sum = __uint_as_float(
          tmem_load_column(tmem_base + ((quarter * 32u) << 16) + acc_stage * kAccColumns));
      ptx::tmem_load_wait();
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbarrier_arrive(&acc_empty[acc_stage]);
      if (++acc_stage == kAccStages) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
      const uint32_t row = row_tile * kTileRows + row_in_tile;
      if (parts == 1u) {
        if (row < n) output[row] = __float2bfloat16_rn(sum * alpha);
        continue;
      }
      // Each warp settles its own 32 rows: no barrier between the warps, one counter per
      // quarter of a row tile.
      partials[part * padded_rows + row] = sum;
      ptx::fence_acq_rel_gpu();
      __syncwarp();
      unsigned int arrived = 0u;
      if (lane == 0) {
        ptx::fence_acq_rel_gpu();
        arrived = atomicAdd(&counters[row_tile * 4u + quarter], 1u);
      }
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (arrived == parts - 1u) {
        ptx::fence_acq_rel_gpu();
        float total = 0.0f;
        for (uint32_t from = 0; from < parts; ++from) total += __ldcg(partials + from * padded_rows + row);
        if (row < n) output[row] = __float2bfloat16_rn(total * alpha);
        if (lane == 0) counters[row_tile * 4u + quarter] = 0u;   // ready for the next launch
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

int create(int n, int k, cudaStream_t stream, Plan** output) {
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->n = n;
  plan->k = k;
  plan->stream = stream;
  plan->row_tiles = (static_cast<uint32_t>(n) + kTileRows - 1u) / kTileRows;
  int device = 0;
  int status = static_cast<int>(cudaGetDevice(&device));
  if (status == 0) {
    status = static_cast<int>(
        cudaDeviceGetAttribute(&plan->sm_count, cudaDevAttrMultiProcessorCount, device));
  }
  if (status == 0) {
    const uint32_t k_stages = (static_cast<uint32_t>(k) + kStageElements - 1u) / kStageElements;
    const uint64_t total = static_cast<uint64_t>(plan->row_tiles) * k_stages;
    plan->grid = total < static_cast<uint64_t>(plan->sm_count) ? static_cast<uint32_t>(total)
                                                              : static_cast<uint32_t>(plan->sm_count);
    plan->max_contributors = 1u;
    for (uint32_t tile = 0; tile < plan->row_tiles; ++tile) {
      const uint64_t begin = static_cast<uint64_t>(tile) * k_stages;
      const uint32_t contributors = owner_of(begin + k_stages - 1u, total, plan->grid) -
                                    owner_of(begin, total, plan->grid) + 1u;
      if (contributors > plan->max_contributors) plan->max_contributors = contributors;
    }
    status = static_cast<int>(cudaHostAlloc(reinterpret_cast<void**>(&plan->status),
                                            sizeof(uint32_t), cudaHostAllocMapped));
  }
  if (status == 0 && plan->max_contributors > 1u) {
    const size_t padded_rows = static_cast<size_t>(plan->row_tiles) * kTileRows;
    status = static_cast<int>(cudaMallocAsync(reinterpret_cast<void**>(&plan->partials),
                                              plan->max_contributors * padded_rows * sizeof(float), stream));
    if (status == 0) {
      status = static_cast<int>(cudaMallocAsync(reinterpret_cast<void**>(&plan->counters),
                                                plan->row_tiles * 4u * sizeof(unsigned int), stream));
    }
    if (status == 0) {
      status = static_cast<int>(
          cudaMemsetAsync(plan->counters, 0, plan->row_tiles * 4u * sizeof(unsigned int), stream));
    }
  }
  if (status == 0) {
    status = static_cast<int>(cudaFuncSetAttribute(
        fp4_vector_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout::kDynamicBytes));
  }
  if (status != 0) {
    destroy(plan);
    return status;
  }
  *plan->status = 0u;
  *output = plan;
  return 0;
}

int execute(Plan* plan, cudaStream_t stream, const void* input, const void* input_scales,
            const void* weight, const void* weight_scales, void* output, float alpha) {
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  if (weight != plan->cached_weight) {
    const int status = encode_k_major_map(&plan->weight_map, weight, static_cast<uint64_t>(plan->n),
                                          static_cast<uint64_t>(plan->k) / 2u, 1u, kTileRows);
    if (status != 0) return status;
    plan->cached_weight = weight;
  }
  if (input != plan->cached_input) {
    const int status = encode_k_major_map(&plan->input_map, input, 1u,
                                          static_cast<uint64_t>(plan->k) / 2u, 1u, kVectorRows);
    if (status != 0) return status;
    plan->cached_input = input;
  }
  fp4_vector_tc_kernel<<<plan->grid, kThreads, Layout::kDynamicBytes, stream>>>(
      plan->weight_map, plan->input_map, static_cast<const uint8_t*>(weight_scales),
      static_cast<const uint8_t*>(input_scales), static_cast<__nv_bfloat16*>(output), plan->partials,
      plan->counters, static_cast<uint32_t>(plan->n), static_cast<uint32_t>(plan->k),
      plan->row_tiles, alpha, plan->status);
  return static_cast<int>(cudaPeekAtLastError());
}

void destroy(Plan* plan) {
  if (plan == nullptr) return;
  if (plan->partials != nullptr) cudaFreeAsync(plan->partials, plan->stream);
  if (plan->counters != nullptr) cudaFreeAsync(plan->counters, plan->stream);
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}

}  // namespace fp4_vector_tc
}  // namespace mircuda_b200
