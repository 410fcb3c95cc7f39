// W4A16 dense projection on the Marlin layout for decode, streaming kernel: bf16 activations
// [tokens <= 16, K] times NVFP4 weights in Marlin tiles with prepared 8-bit group-16 scales
// (marlin_prepare.cu), to bf16 [tokens, N]. Used by mircuda_marlin_nvfp4_dense_execute
// (marlin_dense.cu) for the shapes it covers; the machine is the one of nvfp4_stream.cu:
//  * one persistent CTA per SM takes units u = cta, cta + grid, ...; a unit is one 64-column
//    tile of N and one slice of K; sixteen consumer warps split the slice's 16-element K tiles
//    (a warp's "part" is two consecutive K tiles of every 32), a seventeenth warp adds their sums.
//    (Units of one 16-column quarter of a tile, which need no K slices for small N, were measured
//    and dropped: 4-byte copies per lane ran at two thirds of the rate of 16-byte ones.);
//  * every lane fetches exactly the bytes it will consume (its 16 bytes of a 512-byte weight
//    tile and the 8 scale bytes of its row pair) with asynchronous copies into a ring of private
//    shared-memory slots, six parts ahead, and waits only for its own copies;
//  * one packed word is one thread's A fragment of mma.sync.m16n8k16 for a 16-row block. Its
//    nibbles are converted in memory order, two per cvt.rn.f16x2.e2m1x2, which places K elements
//    (2q, 2q+8) and (2q+1, 2q+9) in the fragment's K slots; the activation fragment is loaded in
//    the same order, so no nibble is moved. A K tile is exactly one scale group, so the MMA runs
//    on unscaled weights and the group scale (prepared code -> f16 bits -> fp32) multiplies the
//    16-element partial sums in fp32;
//  * activations are converted bf16 -> f16 (saturating at +-65504, exact from 2^-14 up) once
//    per unit and stay in registers;
//  * K slices of one N tile meet in the caller's `temporary` buffer: the slice that arrives last
//    (a counter in the caller's `locks`, back to zero when the launch ends) adds them in slice
//    order. When a slice is longer than the fragments a warp can hold, the CTA makes several
//    passes over its units and the reducer keeps running sums in shared memory.
// Numerics against the reference's kernel (sys/native/marlin/vendor/dense_template.h:1655-1658):
// the same exact weight values and scales, fp32 accumulation, the prepared global scale applied
// before the bf16 round; the order of the fp32 additions differs.
// The only waits are on shared-memory barriers between the consumers and the reducer of a CTA,
// and they are bounded.
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>

#include "marlin_stream.hpp"
#include "ptx.cuh"

namespace mircuda_b200 {
namespace marlin_stream {

constexpr int kConsumerWarps = 16;
constexpr int kReducerWarp = kConsumerWarps;
constexpr int kThreads = (kConsumerWarps + 1) * 32;          // 544
constexpr int kTileN = 64;
constexpr int kTileK = 16;
constexpr int kMaxTokens = 16;

// ROW_GROUPS: 1 for up to 8 tokens, 2 for up to 16.
constexpr int kPartTiles = 2;                                // K tiles of a warp's part
constexpr int kPartK = kConsumerWarps * kPartTiles * kTileK; // 512
constexpr int kSlotWeightBytes = kPartTiles * 32 * 16;       // 1024
constexpr int kSlotScaleBytes = kPartTiles * 32 * 8;         // 512
constexpr int kSlotBytes = kSlotWeightBytes + kSlotScaleBytes;
constexpr int kMaxUnitsPerCta = 4;                           // running sums kept across passes

template <int ROW_GROUPS>
struct Geometry {
  static constexpr int kDepth = ROW_GROUPS == 1 ? 6 : 5;               // parts in flight per warp
  static constexpr int kTokens = 8 * ROW_GROUPS;
  static constexpr int kUnitOutputs = kTileN * kTokens;
  static constexpr int kPieces = kUnitOutputs / 4 / 32;                // float4 per reducer lane
  static constexpr int kWarpRingBytes = kDepth * kSlotBytes;
  static constexpr int kRings = 0;
  static constexpr int kSums = kRings + kConsumerWarps * kWarpRingBytes;    // [warp][row][token]
  static constexpr int kRunning = kSums + kConsumerWarps * kUnitOutputs * 4;
  static constexpr int kBarriers = kRunning + kMaxUnitsPerCta * kUnitOutputs * 4;
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

// The two f16 halves of a word as fp32.
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

// d = a * b with a zero accumulator going in.
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

__device__ __forceinline__ void store_shared_float4(uint32_t address, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(address), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
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

// K tile of (slice, pass, part, warp, j): the slice's tiles in order, parts of 32 tiles, two per warp.
template <int ROW_GROUPS, int CPW>
__global__ void __launch_bounds__(kThreads, 1)
marlin_stream_kernel(const __nv_bfloat16* __restrict__ input, const uint8_t* __restrict__ weight,
                     const uint8_t* __restrict__ scales, const float* __restrict__ global_scale,
                     __nv_bfloat16* __restrict__ output, float* __restrict__ temporary,
                     int* __restrict__ locks, int tokens, int n, int k, int slices, int passes,
                     uint32_t* __restrict__ status) {
  using G = Geometry<ROW_GROUPS>;
  constexpr int kDepth = G::kDepth;
  constexpr int kTokens = G::kTokens;
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
  const int units = tiles_n * slices;
  const int my_units = cta < units ? (units - cta + grid - 1) / grid : 0;

  // Programmatic dependent launch (a no-op unless the launch asked for it): weights and their
  // scales are taken to be constant and are fetched at once; activations, outputs, `temporary`
  // and `locks` are only touched after the kernel before this one has completed.
  ptx::dependency_launch_next();
  if (threadIdx.x == kReducerWarp * 32) {
    ptx::mbarrier_init(sums_full, kConsumerWarps);
    ptx::mbarrier_init(sums_empty, 1);
    *abort = 0u;
    ptx::fence_barrier_init();
  }

  if (warp == kReducerWarp) {
    // ---------------------------------------------------------------------- reducer
    __syncthreads();
    ptx::dependency_wait();
    constexpr int kPieces = G::kPieces;
    constexpr int kPiecesPerRow = kTokens / 4;              // 2 or 4
    // prepared global = global * 2^119 / factor; the weights carry factor * 128.
    const float finish = *global_scale * 1.17549435082228751e-38f;   // 2^-126
    uint32_t phase = 0;
    bool alive = true;
    for (int pass = 0; alive && pass < passes; ++pass) {
      for (int unit_index = 0; unit_index < my_units; ++unit_index) {
        if (!__all_sync(0xffffffffu, ptx::mbarrier_wait(sums_full, phase, abort))) {
          alive = false;
          break;
        }
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
        if (passes > 1) {
          const uint32_t running = shared_base + G::kRunning + unit_index * G::kUnitOutputs * 4 + lane * 16;
          if (pass > 0) {
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) {
              add_to(total[piece], load_shared_float4(running + piece * 512));
            }
          }
          if (pass + 1 < passes) {
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) store_shared_float4(running + piece * 512, total[piece]);
            continue;
          }
        }
        const int unit = cta + unit_index * grid;
        const int tile_n = unit % tiles_n;
        if (slices > 1) {
          // Hand-over between the K slices of this N tile: [slice][tile][piece] in `temporary`.
          const int slice = unit / tiles_n;
          float4* mine = reinterpret_cast<float4*>(temporary) +
                         (static_cast<size_t>(slice) * tiles_n + tile_n) * (G::kUnitOutputs / 4) + lane;
#pragma unroll
          for (int piece = 0; piece < kPieces; ++piece) mine[piece * 32] = total[piece];
          ptx::fence_acq_rel_gpu();
          __syncwarp();
          int arrived = 0;
          if (lane == 0) arrived = atomicAdd(&locks[tile_n], 1);
          arrived = __shfl_sync(0xffffffffu, arrived, 0);
          if (arrived != slices - 1) continue;
          if (lane == 0) locks[tile_n] = 0;
          ptx::fence_acq_rel_gpu();
          const float4* first = reinterpret_cast<const float4*>(temporary) +
                                static_cast<size_t>(tile_n) * (G::kUnitOutputs / 4) + lane;
#pragma unroll
          for (int piece = 0; piece < kPieces; ++piece) total[piece] = __ldcg(first + piece * 32);
          for (int other = 1; other < slices; ++other) {
            const float4* next = first + static_cast<size_t>(other) * tiles_n * (G::kUnitOutputs / 4);
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) add_to(total[piece], __ldcg(next + piece * 32));
          }
        }
#pragma unroll
        for (int piece = 0; piece < kPieces; ++piece) {
          const int index = piece * 32 + lane;
          const int row = index / kPiecesPerRow;
          const int token = (index % kPiecesPerRow) * 4;
          const float values[4] = {total[piece].x, total[piece].y, total[piece].z, total[piece].w};
#pragma unroll
          for (int item = 0; item < 4; ++item) {
            if (token + item < tokens) {
              output[static_cast<size_t>(token + item) * n + tile_n * kTileN + row] =
                  __float2bfloat16_rn(values[item] * finish);
            }
          }
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- consumers
    const int group = lane >> 2;
    const int quad = lane & 3;
    const uint32_t ring = shared_base + G::kRings + warp * G::kWarpRingBytes + lane * 16;
    // A slot: the lane's 16 bytes of two weight tiles (2 x 512 bytes), then its 8 scale bytes
    // of the two tiles (2 x 256 bytes); relative to `ring` the scale bytes sit at:
    const uint32_t scale_slot = kSlotWeightBytes - lane * 8;
    const uint32_t tile_row_bytes = static_cast<uint32_t>(tiles_n) * 512u;   // one K tile of all N tiles
    const uint8_t* const lane_weight = weight + static_cast<size_t>(warp) * kPartTiles * tile_row_bytes + lane * 16;
    const uint8_t* const lane_scale = scales + static_cast<size_t>(warp) * kPartTiles * n + group * 8;

    // Fetch cursor: the part that goes into the ring next, as byte offsets from `lane_weight` and
    // `lane_scale` (the operands are smaller than 4 GB, see prepare()). A part is 32 K tiles
    // further on than the one before; the division only happens when a new unit starts.
    int ahead_pass = 0, ahead_unit = 0, ahead_part = 0;
    uint32_t ahead_weight = 0u, ahead_scale = 0u;
    auto locate = [&]() {
      const int unit = cta + ahead_unit * grid;
      const int tile_n = unit % tiles_n;
      const int slice = unit / tiles_n;
      const uint32_t first_tile =
          static_cast<uint32_t>((slice * passes + ahead_pass) * CPW) * (kConsumerWarps * kPartTiles);
      ahead_weight = first_tile * tile_row_bytes + static_cast<uint32_t>(tile_n) * 512u;
      ahead_scale = first_tile * static_cast<uint32_t>(n) + static_cast<uint32_t>(tile_n) * kTileN;
    };
    auto fetch = [&](uint32_t slot) {
      if (ahead_pass < passes) {
        const uint8_t* source = lane_weight + ahead_weight;
        const uint8_t* scale = lane_scale + ahead_scale;
        const uint32_t destination = ring + slot * kSlotBytes;
        copy_async_16(destination, source);
        copy_async_16(destination + 512, source + tile_row_bytes);
        copy_async_8(destination + scale_slot, scale);
        copy_async_8(destination + scale_slot + 256, scale + n);
        ahead_weight += (kConsumerWarps * kPartTiles) * tile_row_bytes;
        ahead_scale += (kConsumerWarps * kPartTiles) * static_cast<uint32_t>(n);
        if (++ahead_part == CPW) {
          ahead_part = 0;
          if (++ahead_unit == my_units) {
            ahead_unit = 0;
            ++ahead_pass;
          }
          locate();
        }
      }
    };
    if (my_units == 0) ahead_pass = passes;
    locate();
#pragma unroll
    for (int slot = 0; slot < kDepth; ++slot) {
      fetch(slot);
      copy_async_commit();
    }
    __syncthreads();
    ptx::dependency_wait();

    uint32_t slot = 0, phase = 0;
    int loaded_slice = -1, loaded_pass = -1;
    bool alive = true;
    uint32_t b[CPW][kPartTiles][ROW_GROUPS][2];
    for (int pass = 0; pass < passes; ++pass) {
      for (int unit_index = 0; unit_index < my_units; ++unit_index) {
        const int unit = cta + unit_index * grid;
        const int slice = unit / tiles_n;
        if (slice != loaded_slice || pass != loaded_pass) {
          // B fragments of this K range: token `group` (+ 8), K elements (2q, 2q+8) and
          // (2q+1, 2q+9) of every tile of this warp, the order the weights decode in.
          loaded_slice = slice;
          loaded_pass = pass;
#pragma unroll
          for (int part = 0; part < CPW; ++part) {
#pragma unroll
            for (int j = 0; j < kPartTiles; ++j) {
              const int element =
                  ((((slice * passes + pass) * CPW + part) * kConsumerWarps + warp) * kPartTiles + j) * kTileK +
                  quad * 2;
#pragma unroll
              for (int rows = 0; rows < ROW_GROUPS; ++rows) {
                uint32_t near = 0u, far = 0u;
                if (rows * 8 + group < tokens) {
                  const __nv_bfloat16* x = input + static_cast<size_t>(rows * 8 + group) * k + element;
                  near = bf16x2_to_f16x2(__ldg(reinterpret_cast<const uint32_t*>(x)));
                  far = bf16x2_to_f16x2(__ldg(reinterpret_cast<const uint32_t*>(x + 8)));
                }
                b[part][j][rows][0] = prmt(near, far, 0x5410u);
                b[part][j][rows][1] = prmt(near, far, 0x7632u);
              }
            }
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
#pragma unroll
          for (int j = 0; j < kPartTiles; ++j) {
            // Prepared scale code c -> f16 bits c << 7. Bytes of rows (g, g + 8) for quarters
            // 0..3 sit at offsets 0,2 | 1,3 | 4,6 | 5,7: even and odd bytes of the two words.
            const uint4 word = load_shared_16(base + j * 512);
            const uint2 scale = load_shared_8(base + scale_slot + j * 256);
            const uint32_t pairs[4] = {(scale.x & 0x00ff00ffu) << 7, (scale.x >> 1) & 0x7f807f80u,
                                       (scale.y & 0x00ff00ffu) << 7, (scale.y >> 1) & 0x7f807f80u};
            const uint32_t quarter_words[4] = {word.x, word.y, word.z, word.w};
#pragma unroll
            for (int quarter = 0; quarter < 4; ++quarter) {
              uint32_t a[4];
              decode_e2m1x8(quarter_words[quarter], a);
              float upper, lower;
              f16x2_to_f32(pairs[quarter], &upper, &lower);
#pragma unroll
              for (int rows = 0; rows < ROW_GROUPS; ++rows) {
                float d[4];
                mma_f16_16x8x16_fresh(d, a, b[part][j][rows][0], b[part][j][rows][1]);
                accumulator[quarter][rows][0] = fmaf(upper, d[0], accumulator[quarter][rows][0]);
                accumulator[quarter][rows][1] = fmaf(upper, d[1], accumulator[quarter][rows][1]);
                accumulator[quarter][rows][2] = fmaf(lower, d[2], accumulator[quarter][rows][2]);
                accumulator[quarter][rows][3] = fmaf(lower, d[3], accumulator[quarter][rows][3]);
              }
            }
          }
          // The part's bytes have been used: refill its slot with the part kDepth further on (one
          // group per part, empty at the end, keeps the wait above counting right).
          fetch(slot);
          copy_async_commit();
          slot = slot + 1 == kDepth ? 0 : slot + 1;
        }
        // This warp's share of the unit: rows quarter * 16 + (group, group + 8), tokens
        // rows * 8 + (2 quad, 2 quad + 1). (Once a wait has run out, `abort` is raised and this
        // lane skips every later wait: the loops run to their end and the launch reports it.)
        if (alive) alive = ptx::mbarrier_wait(sums_empty, phase ^ 1u, abort);
        __syncwarp();
        const uint32_t sums = shared_base + G::kSums + warp * (G::kUnitOutputs * 4);
#pragma unroll
        for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
          for (int rows = 0; rows < ROW_GROUPS; ++rows) {
            const uint32_t address = sums + ((quarter * 16 + group) * kTokens + rows * 8 + quad * 2) * 4;
            store_shared_float2(address, accumulator[quarter][rows][0], accumulator[quarter][rows][1]);
            store_shared_float2(address + 8 * kTokens * 4, accumulator[quarter][rows][2],
                                accumulator[quarter][rows][3]);
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbarrier_arrive(sums_full);
        phase ^= 1u;
      }
    }
    copy_async_wait<0>();      // nothing of this CTA is in flight when it leaves
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort != 0u && status != nullptr) *status = 1u;
}

using Kernel = void (*)(const __nv_bfloat16*, const uint8_t*, const uint8_t*, const float*, __nv_bfloat16*,
                        float*, int*, int, int, int, int, int, uint32_t*);

// The instantiations: a 544-thread CTA has 96 registers per thread, which bounds the activation
// fragments a warp can hold (4 * ROW_GROUPS registers per part).
static Kernel pick(int row_groups, int chunks) {
  if (row_groups == 1) {
    switch (chunks) {
      case 1: return marlin_stream_kernel<1, 1>;
      case 2: return marlin_stream_kernel<1, 2>;
      case 3: return marlin_stream_kernel<1, 3>;
      case 4: return marlin_stream_kernel<1, 4>;
      case 6: return marlin_stream_kernel<1, 6>;
      case 8: return marlin_stream_kernel<1, 8>;
      default: return nullptr;
    }
  }
  switch (chunks) {
    case 1: return marlin_stream_kernel<2, 1>;
    case 2: return marlin_stream_kernel<2, 2>;
    default: return nullptr;
  }
}

static int shared_bytes(int row_groups) {
  return row_groups == 1 ? Geometry<1>::kBytes : Geometry<2>::kBytes;
}

int prepare(Config* config, int tokens, int n, int k, int sm_count) {
  if (tokens <= 0 || tokens > kMaxTokens || n <= 0 || k <= 0 || n % kTileN != 0 || k % kPartK != 0 ||
      static_cast<long long>(n) * k / 2 >= (1ll << 32)) {      // byte offsets are 32-bit in the kernel
    return -1;
  }
  const int row_groups = tokens <= 8 ? 1 : 2;
  const int token_slots = 8 * row_groups;
  const int parts = k / kPartK;
  const int tiles_n = n / kTileN;
  const long long capacity = static_cast<long long>(sm_count) * 4096;    // floats of `temporary`
  // Cost of a split in the time a CTA needs for one part: rounds of units x (parts per unit +
  // start and finish of a unit), plus the hand-over between slices (store, fence, counter,
  // re-read: a chain of L2 round trips, about three parts long as measured).
  const double unit_cost = 0.6, handover_cost = 3.0;
  double best = -1.0;
  for (int slices = 1; slices <= parts; ++slices) {
    if (parts % slices != 0) continue;
    // K slices: one lock per N tile (the caller provides one per SM), partial sums inside
    // `temporary`.
    if (slices > 1 && (tiles_n > sm_count || static_cast<long long>(slices) * n * token_slots > capacity)) {
      continue;
    }
    const int per_unit = parts / slices;
    int chunks = 0;
    for (int candidate = row_groups == 1 ? 8 : 2; candidate >= 1; --candidate) {
      if (per_unit % candidate == 0 && pick(row_groups, candidate) != nullptr) {
        chunks = candidate;
        break;
      }
    }
    if (chunks == 0) continue;
    const int units = tiles_n * slices;
    const int ctas = units < sm_count ? units : sm_count;
    const int rounds = (units + ctas - 1) / ctas;
    const int passes = per_unit / chunks;
    if (passes > 1 && rounds > kMaxUnitsPerCta) continue;
    const double cost = rounds * (per_unit + unit_cost * passes) + (slices > 1 ? handover_cost : 0.0);
    if (best < 0.0 || cost < best - 1e-9) {
      best = cost;
      config->row_groups = row_groups;
      config->chunks_per_warp = chunks;
      config->slices = slices;
      config->passes = passes;
      config->ctas = ctas;
    }
  }
  if (best < 0.0) return -1;
  // The shared-memory attribute is set once per kernel, device and thread.
  static thread_local int configured_device = -1;
  static thread_local unsigned configured = 0u;      // bit = row_groups * 16 + chunks
  int device = 0;
  int status = static_cast<int>(cudaGetDevice(&device));
  if (status != 0) return status;
  if (device != configured_device) {
    configured_device = device;
    configured = 0u;
  }
  const unsigned bit = 1u << ((config->row_groups - 1) * 16 + config->chunks_per_warp);
  if ((configured & bit) == 0u) {
    status = static_cast<int>(cudaFuncSetAttribute(pick(config->row_groups, config->chunks_per_warp),
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   shared_bytes(config->row_groups)));
    if (status != 0) return status;
    configured |= bit;
  }
  return 0;
}

int launch(const Config& config, cudaStream_t stream, bool overlap_launches, const void* input,
           const void* weight, const void* scales, const float* global_scale, void* output,
           void* temporary, void* locks, int tokens, int n, int k, uint32_t* status) {
  cudaLaunchConfig_t launch_config = {};
  launch_config.gridDim = dim3(config.ctas, 1, 1);
  launch_config.blockDim = dim3(kThreads, 1, 1);
  launch_config.dynamicSmemBytes = shared_bytes(config.row_groups);
  launch_config.stream = stream;
  cudaLaunchAttribute attributes[1] = {};
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  launch_config.attrs = attributes;
  launch_config.numAttrs = overlap_launches ? 1 : 0;
  return static_cast<int>(cudaLaunchKernelEx(
      &launch_config, pick(config.row_groups, config.chunks_per_warp),
      static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight),
      static_cast<const uint8_t*>(scales), global_scale, static_cast<__nv_bfloat16*>(output),
      static_cast<float*>(temporary), static_cast<int*>(locks), tokens, n, k, config.slices,
      config.passes, status));
}

}  // namespace marlin_stream
}  // namespace mircuda_b200
