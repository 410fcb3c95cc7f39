// Routed W4A16 projections on the Marlin layout, streaming kernel: the machine of
// marlin_stream.cu for mircuda_marlin_{nvfp4,mxfp4}_moe_execute (marlin_moe.cu) where K is a
// multiple of 256 and at most 2048.
//  * one persistent 544-thread CTA per SM takes units u = cta, cta + grid, ...; a unit is one
//    64-column tile of N and one group of routed rows that share an expert (the 8 rows of a small
//    route block, or 16 of the 64 rows of a large one); the number of units follows from
//    `padded[0]`, which only the device knows;
//  * sixteen consumer warps split K: warp w takes K tile w of every 16 (a "part"), fetching its
//    own 16 bytes of every 512-byte weight tile and the 8 scale bytes of its row pair with
//    asynchronous copies into a ring of private shared-memory slots ten or twelve parts deep;
//  * nibbles are converted in memory order by cvt.rn.f16x2.e2m1x2 and the activation fragment
//    (gathered from the unit's routed token rows, bf16 -> f16) is loaded in the matching order;
//    a K tile lies inside one scale group, so the MMA runs on unscaled weights and the group
//    scale (NVFP4: prepared code -> f16 bits -> fp32; MXFP4: E8M0 byte -> fp32 power of two,
//    clamped to 2^-64 .. 2^63 as in the tile kernel) multiplies the 16-element partial sums;
//  * a seventeenth warp adds the warps' sums of a finished unit, applies the expert's prepared
//    global scale (NVFP4) and the routing weight if asked, and writes one output row per
//    assignment id.
// Nothing is fetched before the kernel in front of this one on the stream has completed: the
// routes it reads are normally that kernel's output. The only waits are on shared-memory
// barriers between the consumers and the reducer of a CTA, and they are bounded.
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "launch_overlap.hpp"
#include "marlin_moe_stream.hpp"
#include "ptx.cuh"

namespace mircuda_b200 {
namespace marlin_moe_stream {

constexpr int kConsumerWarps = 16;
constexpr int kReducerWarp = kConsumerWarps;
constexpr int kThreads = (kConsumerWarps + 1) * 32;          // 544
constexpr int kTileN = 64;
constexpr int kTileK = 16;
constexpr int kPartK = kConsumerWarps * kTileK;              // 256
constexpr int kSlotBytes = 32 * 16 + 32 * 8;                 // a lane's 16 weight and 8 scale bytes
constexpr int kMaxParts = 8;                                 // K <= 2048

template <int ROW_GROUPS>
struct Geometry {
  static constexpr int kDepth = ROW_GROUPS == 1 ? 12 : 10;             // parts in flight per warp
  static constexpr int kRows = 8 * ROW_GROUPS;                         // routed rows of a unit
  static constexpr int kUnitOutputs = kTileN * kRows;
  static constexpr int kPieces = kUnitOutputs / 4 / 32;                // float4 per reducer lane
  static constexpr int kWarpRingBytes = kDepth * kSlotBytes;
  static constexpr int kRings = 0;
  static constexpr int kSums = kRings + kConsumerWarps * kWarpRingBytes;    // [warp][column][row]
  static constexpr int kBarriers = kSums + kConsumerWarps * kUnitOutputs * 4;
  static constexpr int kAbort = kBarriers + 16;
  static constexpr int kBytes = kAbort + 16;
  static_assert(kBytes <= 232448, "fits the shared memory of one SM");
};

__device__ __forceinline__ void decode_e2m1x8(uint32_t codes, uint32_t (&out)[4]) {
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t"
      "}\n"
      : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3])
      : "r"(codes));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

__device__ __forceinline__ void f16x2_to_f32(uint32_t pair, float* low, float* high) {
  asm("{\n\t"
      ".reg .b16 l, h;\n\t"
      "mov.b32 {l, h}, %2;\n\t"
      "cvt.f32.f16 %0, l;\n\t"
      "cvt.f32.f16 %1, h;\n\t"
      "}\n"
      : "=f"(*low), "=f"(*high)
      : "r"(pair));
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t pair) {
  uint32_t d;
  const float low = __uint_as_float(pair << 16);
  const float high = __uint_as_float(pair & 0xffff0000u);
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(high), "f"(low));
  return d;
}

__device__ __forceinline__ void mma_f16_16x8x16_fresh(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                      uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ uint4 load_shared_16(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(address)
               : "memory");
  return v;
}

__device__ __forceinline__ uint2 load_shared_8(uint32_t address) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(address) : "memory");
  return v;
}

__device__ __forceinline__ float4 load_shared_float4(uint32_t address) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(address)
               : "memory");
  return v;
}

__device__ __forceinline__ void store_shared_float2(uint32_t address, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(address), "f"(x), "f"(y) : "memory");
}

__device__ __forceinline__ void copy_async_16(uint32_t destination, const void* source) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(destination), "l"(source) : "memory");
}

__device__ __forceinline__ void copy_async_8(uint32_t destination, const void* source) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(destination), "l"(source) : "memory");
}

__device__ __forceinline__ void copy_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int Pending>
__device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(Pending) : "memory");
}

__device__ __forceinline__ void mbarrier_arrive_after(uint32_t barrier, uint32_t token) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(barrier), "r"(token) : "memory");
}

__device__ __forceinline__ void add_to(float4& total, const float4& v) {
  total.x += v.x;
  total.y += v.y;
  total.z += v.z;
  total.w += v.w;
}

// Two scale bytes in the halves of `pair` (bits 0-7 and 16-23) as fp32 multipliers.
template <bool MXFP4>
__device__ __forceinline__ void scale_pair(uint32_t pair, float* upper, float* lower) {
  if (MXFP4) {
    // E8M0: 2^(e - 127), exponent clamped to 2^-64 .. 2^63
    const uint32_t first = min(max(pair & 0xffu, 63u), 190u);
    const uint32_t second = min(max((pair >> 16) & 0xffu, 63u), 190u);
    *upper = __uint_as_float(first << 23);
    *lower = __uint_as_float(second << 23);
  } else {
    // prepared code c = bits 14:7 of an f16
    f16x2_to_f32(pair << 7, upper, lower);
  }
}

template <int ROW_GROUPS, int CPW, bool MXFP4>
__global__ void __launch_bounds__(kThreads, 1)
marlin_moe_stream_kernel(const __nv_bfloat16* __restrict__ input, const uint8_t* __restrict__ weight,
                         const uint8_t* __restrict__ scales, const float* __restrict__ global_scales,
                         __nv_bfloat16* __restrict__ output, const int* __restrict__ sorted,
                         const int* __restrict__ expert_ids, const int* __restrict__ padded,
                         const float* __restrict__ routing, int top_k, bool multiply_routing, int assignments,
                         int n, int k, int block_size, uint32_t* __restrict__ status) {
  using G = Geometry<ROW_GROUPS>;
  constexpr int kDepth = G::kDepth;
  constexpr int kRows = G::kRows;
  extern __shared__ __align__(16) uint8_t shared[];
  const uint32_t shared_base = ptx::smem_address(shared);
  uint64_t* sums_full = reinterpret_cast<uint64_t*>(shared + G::kBarriers);
  uint64_t* sums_empty = sums_full + 1;
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(shared + G::kAbort);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grid = static_cast<int>(gridDim.x);
  const int cta = static_cast<int>(blockIdx.x);
  const int tiles_n = n / kTileN;

  ptx::dependency_launch_next();
  if (threadIdx.x == kReducerWarp * 32) {
    ptx::mbarrier_init(sums_full, kConsumerWarps);
    ptx::mbarrier_init(sums_empty, 1);
    *abort = 0u;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  ptx::dependency_wait();
  // Row groups of kRows rows up to the padded length, times the N tiles; unit = tile + group * tiles.
  const int units = ((__ldg(padded) + kRows - 1) / kRows) * tiles_n;
  const int my_units = cta < units ? (units - cta + grid - 1) / grid : 0;
  constexpr int kScaleGroupTiles = MXFP4 ? 2 : 1;            // K tiles per scale group
  const size_t expert_weight_bytes = static_cast<size_t>(k / kTileK) * tiles_n * 512;
  const size_t expert_scale_bytes = static_cast<size_t>(n) * (k / kTileK / kScaleGroupTiles);

  if (warp == kReducerWarp) {
    // ---------------------------------------------------------------------- reducer
    constexpr int kPieces = G::kPieces;
    constexpr int kPiecesPerColumn = kRows / 4;              // 2 or 4
    uint32_t phase = 0;
    for (int unit_index = 0; unit_index < my_units; ++unit_index) {
      const int unit = cta + unit_index * grid;
      const int tile_n = unit % tiles_n;
      const int first_row = (unit / tiles_n) * kRows;
      const int expert = __ldg(expert_ids + first_row / block_size);
      // NVFP4: prepared global = global * 2^119 / factor and the weights carry factor * 128.
      float finish = 1.0f;
      if (!MXFP4 && expert >= 0) finish = __ldg(global_scales + expert) * 1.17549435082228751e-38f;   // 2^-126
      if (!__all_sync(0xffffffffu, ptx::mbarrier_wait(sums_full, phase, abort))) break;
      float4 total[kPieces];
#pragma unroll
      for (int piece = 0; piece < kPieces; ++piece) {
        const uint32_t source = shared_base + G::kSums + (piece * 32 + lane) * 16;
        total[piece] = load_shared_float4(source);
#pragma unroll
        for (int other = 1; other < kConsumerWarps; ++other) {
          add_to(total[piece], load_shared_float4(source + other * G::kUnitOutputs * 4));
        }
      }
      __syncwarp();
      if (lane == 0) mbarrier_arrive_after(ptx::smem_address(sums_empty), __float_as_uint(total[0].x));
      phase ^= 1u;
      if (expert < 0) continue;
#pragma unroll
      for (int piece = 0; piece < kPieces; ++piece) {
        const int index = piece * 32 + lane;
        const int column = index / kPiecesPerColumn;
        const int row = (index % kPiecesPerColumn) * 4;
        const float values[4] = {total[piece].x, total[piece].y, total[piece].z, total[piece].w};
#pragma unroll
        for (int item = 0; item < 4; ++item) {
          const int id = __ldg(sorted + first_row + row + item);
          if (id < assignments) {
            float value = values[item] * finish;
            if (multiply_routing) value *= __ldg(routing + id);
            output[static_cast<size_t>(id) * n + tile_n * kTileN + column] = __float2bfloat16_rn(value);
          }
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- consumers
    const int group = lane >> 2;
    const int quad = lane & 3;
    const uint32_t ring = shared_base + G::kRings + warp * G::kWarpRingBytes + lane * 16;
    // A slot: the lane's 16 bytes of a weight tile (512 bytes for the warp), then its 8 scale
    // bytes (256 bytes); relative to `ring` the scale bytes sit at:
    const uint32_t scale_slot = 512u - lane * 8u;
    const uint32_t tile_row_bytes = static_cast<uint32_t>(tiles_n) * 512u;   // one K tile of all N tiles
    const uint32_t lane_weight = static_cast<uint32_t>(warp) * tile_row_bytes + lane * 16;
    const uint32_t lane_scale = static_cast<uint32_t>(warp / kScaleGroupTiles) * n + group * 8;
    const uint32_t weight_part_stride = kConsumerWarps * tile_row_bytes;
    const uint32_t scale_part_stride = (kConsumerWarps / kScaleGroupTiles) * static_cast<uint32_t>(n);

    // Fetch cursor: the part that goes into the ring next (byte offsets inside the unit's expert).
    int ahead_unit = 0, ahead_part = 0;
    const uint8_t* ahead_weight = weight;
    const uint8_t* ahead_scale = scales;
    auto locate = [&]() {
      if (ahead_unit >= my_units) return;
      const int unit = cta + ahead_unit * grid;
      const int tile_n = unit % tiles_n;
      const int first_row = (unit / tiles_n) * kRows;
      int expert = __ldg(expert_ids + first_row / block_size);
      if (expert < 0) expert = 0;          // a block without an expert: its sums are not written
      ahead_weight = weight + static_cast<size_t>(expert) * expert_weight_bytes + lane_weight + tile_n * 512;
      ahead_scale = scales + static_cast<size_t>(expert) * expert_scale_bytes + lane_scale + tile_n * kTileN;
    };
    auto fetch = [&](uint32_t slot) {
      if (ahead_unit < my_units) {
        const uint32_t destination = ring + slot * kSlotBytes;
        copy_async_16(destination, ahead_weight);
        copy_async_8(destination + scale_slot, ahead_scale);
        ahead_weight += weight_part_stride;
        ahead_scale += scale_part_stride;
        if (++ahead_part == CPW) {
          ahead_part = 0;
          ++ahead_unit;
          locate();
        }
      }
    };
    locate();
#pragma unroll
    for (int slot = 0; slot < kDepth; ++slot) {
      fetch(slot);
      copy_async_commit();
    }

    uint32_t slot = 0, phase = 0;
    bool alive = true;
    for (int unit_index = 0; unit_index < my_units; ++unit_index) {
      const int unit = cta + unit_index * grid;
      const int first_row = (unit / tiles_n) * kRows;
      // B fragments: routed row `group` (+ 8) of the unit, K elements (2q, 2q+8) and (2q+1, 2q+9)
      // of every K tile of this warp, the order the weights decode in.
      uint32_t b[CPW][ROW_GROUPS][2];
#pragma unroll
      for (int rows = 0; rows < ROW_GROUPS; ++rows) {
        const int id = __ldg(sorted + first_row + rows * 8 + group);
        const __nv_bfloat16* x = input + static_cast<size_t>(id < assignments ? id / top_k : 0) * k +
                                 warp * kTileK + quad * 2;
#pragma unroll
        for (int part = 0; part < CPW; ++part) {
          uint32_t near = 0u, far = 0u;
          if (id < assignments) {
            near = bf16x2_to_f16x2(__ldg(reinterpret_cast<const uint32_t*>(x + part * kPartK)));
            far = bf16x2_to_f16x2(__ldg(reinterpret_cast<const uint32_t*>(x + part * kPartK + 8)));
          }
          b[part][rows][0] = prmt(near, far, 0x5410u);
          b[part][rows][1] = prmt(near, far, 0x7632u);
        }
      }
      float accumulator[4][ROW_GROUPS][4];
#pragma unroll
      for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
        for (int rows = 0; rows < ROW_GROUPS; ++rows) {
#pragma unroll
          for (int item = 0; item < 4; ++item) accumulator[quarter][rows][item] = 0.0f;
        }
      }
#pragma unroll
      for (int part = 0; part < CPW; ++part) {
        copy_async_wait<kDepth - 1>();       // this lane's copies of the oldest part have landed
        const uint32_t base = ring + slot * kSlotBytes;
        const uint4 word = load_shared_16(base);
        const uint2 scale = load_shared_8(base + scale_slot);
        // Scale bytes of rows (g, g + 8) for quarters 0..3 sit at offsets 0,2 | 1,3 | 4,6 | 5,7:
        // even and odd bytes of the two words.
        const uint32_t pairs[4] = {scale.x & 0x00ff00ffu, (scale.x >> 8) & 0x00ff00ffu, scale.y & 0x00ff00ffu,
                                   (scale.y >> 8) & 0x00ff00ffu};
        const uint32_t quarter_words[4] = {word.x, word.y, word.z, word.w};
#pragma unroll
        for (int quarter = 0; quarter < 4; ++quarter) {
          uint32_t a[4];
          decode_e2m1x8(quarter_words[quarter], a);
          float upper, lower;
          scale_pair<MXFP4>(pairs[quarter], &upper, &lower);
#pragma unroll
          for (int rows = 0; rows < ROW_GROUPS; ++rows) {
            float d[4];
            mma_f16_16x8x16_fresh(d, a, b[part][rows][0], b[part][rows][1]);
            accumulator[quarter][rows][0] = fmaf(upper, d[0], accumulator[quarter][rows][0]);
            accumulator[quarter][rows][1] = fmaf(upper, d[1], accumulator[quarter][rows][1]);
            accumulator[quarter][rows][2] = fmaf(lower, d[2], accumulator[quarter][rows][2]);
            accumulator[quarter][rows][3] = fmaf(lower, d[3], accumulator[quarter][rows][3]);
          }
        }
        // The part's bytes have been used: refill its slot with the part kDepth further on (one
        // group per part, empty at the end, keeps the wait above counting right).
        fetch(slot);
        copy_async_commit();
        slot = slot + 1 == kDepth ? 0 : slot + 1;
      }
      // This warp's share of the unit: columns quarter * 16 + (group, group + 8), routed rows
      // rows * 8 + (2 quad, 2 quad + 1). (Once a wait has run out, `abort` is raised and this lane
      // skips every later wait: the loops run to their end and the launch reports it.)
      if (alive) alive = ptx::mbarrier_wait(sums_empty, phase ^ 1u, abort);
      __syncwarp();
      const uint32_t sums = shared_base + G::kSums + warp * (G::kUnitOutputs * 4);
#pragma unroll
      for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
        for (int rows = 0; rows < ROW_GROUPS; ++rows) {
          const uint32_t address = sums + ((quarter * 16 + group) * kRows + rows * 8 + quad * 2) * 4;
          store_shared_float2(address, accumulator[quarter][rows][0], accumulator[quarter][rows][1]);
          store_shared_float2(address + 8 * kRows * 4, accumulator[quarter][rows][2], accumulator[quarter][rows][3]);
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbarrier_arrive(sums_full);
      phase ^= 1u;
    }
    copy_async_wait<0>();      // nothing of this CTA is in flight when it leaves
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort != 0u && status != nullptr) *status = 1u;
}

using Kernel = void (*)(const __nv_bfloat16*, const uint8_t*, const uint8_t*, const float*, __nv_bfloat16*,
                        const int*, const int*, const int*, const float*, int, bool, int, int, int, int,
                        uint32_t*);

template <int ROW_GROUPS, bool MXFP4>
Kernel pick(int parts) {
  switch (parts) {
    case 1: return marlin_moe_stream_kernel<ROW_GROUPS, 1, MXFP4>;
    case 2: return marlin_moe_stream_kernel<ROW_GROUPS, 2, MXFP4>;
    case 3: return marlin_moe_stream_kernel<ROW_GROUPS, 3, MXFP4>;
    case 4: return marlin_moe_stream_kernel<ROW_GROUPS, 4, MXFP4>;
    case 5: return marlin_moe_stream_kernel<ROW_GROUPS, 5, MXFP4>;
    case 6: return marlin_moe_stream_kernel<ROW_GROUPS, 6, MXFP4>;
    case 7: return marlin_moe_stream_kernel<ROW_GROUPS, 7, MXFP4>;
    default: return marlin_moe_stream_kernel<ROW_GROUPS, 8, MXFP4>;
  }
}

bool eligible(int n, int k) { return n > 0 && n % kTileN == 0 && k > 0 && k % kPartK == 0 && k / kPartK <= kMaxParts; }

int launch(cudaStream_t stream, bool mxfp4, int block_size, const void* input, const void* weight,
           const void* scales, const void* global_scales, void* output, const void* sorted, const void* expert_ids,
           const void* padded, const void* routing, int top_k, bool multiply_routing, int assignments, int n,
           int k, uint32_t* status) {
  if (!eligible(n, k)) return -1;
  const int row_groups = block_size == 8 ? 1 : 2;
  const int parts = k / kPartK;
  Kernel kernel = row_groups == 1 ? (mxfp4 ? pick<1, true>(parts) : pick<1, false>(parts))
                                  : (mxfp4 ? pick<2, true>(parts) : pick<2, false>(parts));
  const int bytes = row_groups == 1 ? Geometry<1>::kBytes : Geometry<2>::kBytes;
  int device = 0, sm_count = 0;
  int result = static_cast<int>(cudaGetDevice(&device));
  if (result == 0) result = static_cast<int>(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  if (result == 0) {
    result = static_cast<int>(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  }
  if (result != 0) return result;
  return launch_after_dependency(kernel, dim3(sm_count), dim3(kThreads), static_cast<size_t>(bytes), stream,
                                 static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
                                 static_cast<const uint8_t*>(scales), static_cast<const float*>(global_scales),
                                 static_cast<__nv_bfloat16*>(output), static_cast<const int*>(sorted),
                                 static_cast<const int*>(expert_ids), static_cast<const int*>(padded),
                                 static_cast<const float*>(routing), top_k, multiply_routing, assignments, n, k,
                                 block_size, status);
}

}  // namespace marlin_moe_stream
}  // namespace mircuda_b200
