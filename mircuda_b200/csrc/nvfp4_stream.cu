// bf16-activation x NVFP4-weight skinny GEMM for decode (M <= 8), streaming kernel:
//   y[m, n] = bf16(global * sum_k x[m, k] * e2m1(W[n, k]) * ue4m3(s[n, k / 16]))
// Same operands and numerics as the kernels in nvfp4_vector.cu (exact weight x scale products
// in f16, activations converted bf16 -> f16, fp32 accumulation in mma.sync); a different
// machine around them, built for a launch that lasts a few microseconds and has to keep HBM
// busy from its first cycle to its last:
//  * one persistent CTA per SM walks over 16-row tiles, tile t of CTA c being c, c + grid, ...;
//    a tile's 16 rows are the rows of one 128-row scale tile that share four 16-byte lines of
//    every scale atom (rows 4L..4L+3 of each 32-row quarter), so the tile's scale bytes are 64
//    contiguous bytes per atom;
//  * sixteen consumer warps each own one 128-element K chunk of every 2048-element stage of a
//    tile, so a warp's activation fragments only change between passes over K: they are loaded
//    and converted once per pass and stay in registers;
//  * there is no producer and no barrier on the way in: every lane fetches exactly the bytes it
//    will consume (16 bytes of two weight rows and the two 4-byte scale words of those rows)
//    with asynchronous copies into a ring of private shared-memory slots, up to eight chunks
//    (a whole number of tiles) ahead, and waits only for its own copies (cp.async groups). Up to
//    160 KB per SM are in flight from the first instruction on; a first version that fed the same consumers by TMA (seventeen
//    64-byte-wide boxes per stage) delivered 2.2 TB/s: too many small requests for the TMA unit;
//  * per chunk a lane issues two 16-byte and two 2-byte shared loads, 32 E2M1 conversions,
//    32 packed multiplies by the block scale and 8 mma.sync; addresses are computed once per
//    tile;
//  * a reducer warp adds the sixteen warps' partial sums of a finished tile (through a
//    four-deep ring of shared buffers, so the consumers never wait for it) and writes the bf16
//    outputs. When K is longer than the activation fragments a warp can hold (3 chunks), the
//    CTA makes several passes over K, each over all of its tiles, and the reducer keeps the
//    tiles' running sums in shared memory: nothing passes through global memory and no
//    hand-over between CTAs exists.
// The only waits are on shared-memory barriers between the consumers and the reducer of a
// CTA, and they are bounded.
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>

#include "nvfp4_stream.hpp"
#include "ptx.cuh"

namespace mircuda_b200 {
namespace nvfp4_stream {

constexpr int kConsumerWarps = 16;
constexpr int kReducerWarp = kConsumerWarps;
constexpr int kThreads = (kConsumerWarps + 1) * 32;          // 544
constexpr int kTileRows = 16;
constexpr int kStageChunks = kConsumerWarps;                 // one 128-element chunk per consumer warp
constexpr int kStageK = kStageChunks * 128;                  // 2048
constexpr int kDepth = 8;                                    // slots of a warp's private ring
constexpr int kSlotWeightBytes = 2 * 32 * 16;                // two row halves x 32 lanes x 16 bytes
constexpr int kSlotScaleBytes = 2 * 32 * 4;                  // two row halves x 32 lanes x 4 bytes
constexpr int kSlotBytes = kSlotWeightBytes + kSlotScaleBytes;       // 1280
constexpr int kWarpRingBytes = kDepth * kSlotBytes;
constexpr int kSumBuffers = 4;
constexpr int kTileOutputs = kTileRows * 8;                  // rows x token slots
constexpr int kSumBufferBytes = kConsumerWarps * kTileOutputs * 4;   // 8 KB
constexpr int kMaxChunksPerWarp = 3;
constexpr int kMaxTilesPerCta = 64;                          // running sums kept across passes

struct SharedLayout {
  static constexpr int kRings = 0;
  static constexpr int kSums = kRings + kConsumerWarps * kWarpRingBytes;
  static constexpr int kRunning = kSums + kSumBuffers * kSumBufferBytes;     // [tile][128] f32
  static constexpr int kBarriers = kRunning + kMaxTilesPerCta * kTileOutputs * 4;
  static constexpr int kAbort = kBarriers + 2 * kSumBuffers * 8;
  static constexpr int kBytes = kAbort + 16;
  static_assert(kBytes <= 232448, "fits the shared memory of one SM");
};

// Four packed bytes of E2M1 codes (even k in the low nibble) -> four f16x2 in K order.
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

// Two UE4M3 scale bytes (the low 16 bits) -> f16x2 (s0, s1), exact; the top bit of a scale
// byte carries no meaning and is dropped.
__device__ __forceinline__ uint32_t decode_scales(uint32_t two_bytes) {
  uint32_t pair;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(static_cast<uint16_t>(two_bytes & 0x7f7fu)));
  return pair;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Two bf16 -> two f16 (round to nearest, saturating at +-65504); exact for magnitudes in
// [2^-14, 65504].
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t pair) {
  uint32_t d;
  const float low = __uint_as_float(pair << 16);
  const float high = __uint_as_float(pair & 0xffff0000u);
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(high), "f"(low));
  return d;
}

__device__ __forceinline__ void mma_f16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1,
                                                uint32_t a2, uint32_t a3, uint32_t b0,
                                                uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_shared_16(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(address)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t load_shared_u16(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(address) : "memory");
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

// Asynchronous copies global -> shared: 16 bytes past L1 (streamed once), 4 bytes through it.
__device__ __forceinline__ void copy_async_16(uint32_t destination, const void* source) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(destination), "l"(source) : "memory");
}

__device__ __forceinline__ void copy_async_4(uint32_t destination, const void* source) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(destination), "l"(source) : "memory");
}

__device__ __forceinline__ void copy_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int Pending>
__device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(Pending) : "memory");
}

// Arrival on a barrier of this CTA, ordered after `token` has been produced (the compiler
// cannot hoist it above the instructions that computed the value).
__device__ __forceinline__ void mbarrier_arrive_after(uint32_t barrier, uint32_t token) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(barrier), "r"(token) : "memory");
}

// Slots of a warp's private ring: a whole number of tiles (CPW chunks each), at most eight.
template <int CPW>
struct Ring {
  static constexpr int kTiles = 8 / CPW;          // tiles in flight per warp: 8, 4, 2
  static constexpr int kSlots = kTiles * CPW;
};

// FP4_INPUT: the activations are one NVFP4 vector (E2M1 codes + swizzled UE4M3 block scales, the
// operands of mircuda_fp4_vector_*) instead of bf16 rows; code x scale is exact in f16, so the
// fragments hold the dequantised vector and everything after them is unchanged.
template <int CPW, bool FP4_INPUT>
__global__ void __launch_bounds__(kThreads, 1)
nvfp4_stream_kernel(const uint8_t* __restrict__ weight, const uint8_t* __restrict__ weight_scales,
                    const void* __restrict__ input_pointer, const uint8_t* __restrict__ input_scales,
                    __nv_bfloat16* __restrict__ output, int m, int n, int k, int tiles, int passes,
                    float global_scale, uint32_t* __restrict__ status) {
  const __nv_bfloat16* input = static_cast<const __nv_bfloat16*>(input_pointer);
  extern __shared__ __align__(16) uint8_t shared[];
  const uint32_t shared_base = ptx::smem_address(shared);
  uint64_t* sums_full = reinterpret_cast<uint64_t*>(shared + SharedLayout::kBarriers);   // [kSumBuffers]
  uint64_t* sums_empty = sums_full + kSumBuffers;                                        // [kSumBuffers]
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(shared + SharedLayout::kAbort);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grid = static_cast<int>(gridDim.x);
  const int cta = static_cast<int>(blockIdx.x);
  const int my_tiles = cta < tiles ? (tiles - cta + grid - 1) / grid : 0;

  // Programmatic dependent launch (a no-op unless the launch asked for it): the next kernel of
  // the stream may be scheduled as soon as every CTA has got here, and this kernel may itself run
  // while the previous one is finishing. Weights and their scales are taken to be constant, so
  // they are fetched at once; every thread that reads activations or writes outputs first waits
  // for the previous kernel to complete.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The barriers between consumers and reducer are set up by the reducer warp while the
  // consumers already issue their first copies; the CTA-wide barrier comes after those.
  if (threadIdx.x == kReducerWarp * 32) {
    for (int buffer = 0; buffer < kSumBuffers; ++buffer) {
      ptx::mbarrier_init(&sums_full[buffer], kConsumerWarps);
      ptx::mbarrier_init(&sums_empty[buffer], 1);
    }
    *abort = 0u;
    ptx::fence_barrier_init();
  }

  if (warp == kReducerWarp) {
    // ---------------------------------------------------------------------- reducer
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t buffer = 0, buffer_phase = 0;
    bool alive = true;
    for (int pass = 0; alive && pass < passes; ++pass) {
      for (int tile_index = 0; tile_index < my_tiles; ++tile_index) {
        if (!__all_sync(0xffffffffu, ptx::mbarrier_wait(&sums_full[buffer], buffer_phase, abort))) {
          alive = false;
          break;
        }
        const uint32_t source = shared_base + SharedLayout::kSums + buffer * kSumBufferBytes + lane * 16;
        float4 total = load_shared_float4(source);
#pragma unroll
        for (int other = 1; other < kConsumerWarps; ++other) {
          const float4 v = load_shared_float4(source + other * kTileOutputs * 4);
          total.x += v.x;
          total.y += v.y;
          total.z += v.z;
          total.w += v.w;
        }
        __syncwarp();
        if (lane == 0) mbarrier_arrive_after(ptx::smem_address(&sums_empty[buffer]), __float_as_uint(total.x));
        if (++buffer == kSumBuffers) {
          buffer = 0;
          buffer_phase ^= 1u;
        }
        if (passes > 1) {
          // Running sums of the tile over the passes; every lane owns its four values.
          const uint32_t running = shared_base + SharedLayout::kRunning + tile_index * kTileOutputs * 4 + lane * 16;
          if (pass > 0) {
            const float4 v = load_shared_float4(running);
            total.x += v.x;
            total.y += v.y;
            total.z += v.z;
            total.w += v.w;
          }
          if (pass + 1 < passes) {
            store_shared_float4(running, total);
            continue;
          }
        }
        // lane -> row lane / 2 of the tile, token slots 4 * (lane % 2) .. + 3
        const int tile = cta + tile_index * grid;
        const int tile_row = lane >> 1;
        const int row = (tile >> 3) * 128 + (tile_row >> 2) * 32 + (tile & 7) * 4 + (tile_row & 3);
        const int token = (lane & 1) * 4;
        const float values[4] = {total.x, total.y, total.z, total.w};
#pragma unroll
        for (int item = 0; item < 4; ++item) {
          if (token + item < m) {
            output[static_cast<size_t>(token + item) * n + row] = __float2bfloat16_rn(values[item] * global_scale);
          }
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- consumers
    const int group = lane >> 2;          // MMA row (and row + 8) / token of the B fragment
    const int quad = lane & 3;
    const int atoms_k = k / 64;
    const size_t row_bytes = static_cast<size_t>(k) / 2;
    const uint32_t ring = shared_base + SharedLayout::kRings + warp * kWarpRingBytes;
    // Tile row i = 4 * quarter + line is row quarter * 32 + 4 * L + line of the 128-row tile;
    // MMA rows `group` and `group + 8` are tile rows i and i + 8 (two quarters = 64 rows on).
    // This lane's 16 bytes of a row are K blocks 2 * quad and 2 * quad + 1 of the warp's chunk;
    // their scale bytes are bytes (quad % 2) * 2 + {0, 1} of the 4-byte word of (atom, row).
    const int row_in_tile = (group >> 2) * 32 + (group & 3);
    const int scale_in_atom = (group & 3) * 16 + (group >> 2) * 4;
    const int total_tiles = passes * my_tiles;
    constexpr int kAhead = Ring<CPW>::kTiles;
    // What does not change from tile to tile: this lane's place inside a tile's rows and inside
    // the warp's chunk of a stage.
    const uint8_t* const lane_weight = weight + static_cast<size_t>(row_in_tile) * row_bytes + warp * 64 + quad * 16;
    const uint8_t* const lane_scale = weight_scales + (warp * 2 + (quad >> 1)) * 512 + scale_in_atom;
    const uint32_t lane_slot = ring + lane * 16;
    // A slot holds the two rows' 16-byte pieces of all lanes (2 x 512 bytes), then their 4-byte
    // scale words (2 x 128 bytes); relative to `lane_slot` this lane's scale words sit at:
    const uint32_t scale_slot = kSlotWeightBytes - lane * 12;

    // Fetches all CPW chunks of one tile of one pass into the ring slots of `ring_tile`.
    auto fetch = [&](int pass, int tile_index, int ring_tile) {
      const int tile = cta + tile_index * grid;
      const int row_tile = tile >> 3, lines = tile & 7;
      const uint8_t* low = lane_weight + static_cast<size_t>(row_tile * 128 + lines * 4) * row_bytes +
                           pass * (CPW * kStageChunks * 64);
      const uint8_t* scale = lane_scale + (static_cast<size_t>(row_tile) * atoms_k + pass * (CPW * kStageChunks * 2)) * 512 +
                             lines * 64;
      uint32_t destination = lane_slot + ring_tile * (CPW * kSlotBytes);
#pragma unroll
      for (int part = 0; part < CPW; ++part) {
        copy_async_16(destination, low);
        copy_async_16(destination + 512, low + 64 * row_bytes);
        copy_async_4(destination + scale_slot, scale);
        copy_async_4(destination + scale_slot + 128, scale + 8);
        destination += kSlotBytes;
        low += kStageChunks * 64;
        scale += kStageChunks * 2 * 512;
      }
    };

    int ahead_pass = 0, ahead_tile = 0, fetched = 0;
#pragma unroll
    for (int ring_tile = 0; ring_tile < kAhead; ++ring_tile) {
      if (fetched < total_tiles) {
        fetch(ahead_pass, ahead_tile, ring_tile);
        ++fetched;
        if (++ahead_tile == my_tiles) {
          ahead_tile = 0;
          ++ahead_pass;
        }
      }
      copy_async_commit();
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float even[4] = {0.0f, 0.0f, 0.0f, 0.0f}, odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    uint32_t ring_tile = 0, buffer = 0, buffer_phase = 0;
    bool alive = true;
    for (int pass = 0; pass < passes; ++pass) {
      // B fragments of this pass: token `group`, this lane's 32 consecutive K-elements of the
      // warp's chunk of every stage, as f16x2 pairs in K order.
      uint32_t b[CPW][16];
#pragma unroll
      for (int part = 0; part < CPW; ++part) {
        const int element = ((pass * CPW + part) * kStageChunks + warp) * 128 + quad * 32;
        if (FP4_INPUT) {
          if (group == 0) {
            // 32 codes (16 bytes) and the two block scales of K blocks element / 16 and + 1: in the
            // one-row swizzled layout block c sits at byte (c / 4) * 512 + c % 4.
            const uint8_t* bytes = static_cast<const uint8_t*>(input_pointer);
            const uint4 codes = __ldg(reinterpret_cast<const uint4*>(bytes + element / 2));
            const int block = element / 16;
            const uint32_t both = decode_scales(
                __ldg(reinterpret_cast<const uint16_t*>(input_scales + (block >> 2) * 512 + (block & 3))));
            const uint32_t multiplier[2] = {prmt(both, both, 0x1010u), prmt(both, both, 0x3232u)};
            const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
            for (int word = 0; word < 4; ++word) {
              uint32_t values[4];
              decode_e2m1x8(words[word], values);
#pragma unroll
              for (int item = 0; item < 4; ++item) {
                b[part][word * 4 + item] = mul_f16x2(values[item], multiplier[word >> 1]);
              }
            }
          } else {
#pragma unroll
            for (int item = 0; item < 16; ++item) b[part][item] = 0u;
          }
        } else if (group < m) {
          const uint4* source = reinterpret_cast<const uint4*>(input + static_cast<size_t>(group) * k + element);
#pragma unroll
          for (int word = 0; word < 4; ++word) {
            const uint4 v = __ldg(source + word);
            b[part][word * 4 + 0] = bf16x2_to_f16x2(v.x);
            b[part][word * 4 + 1] = bf16x2_to_f16x2(v.y);
            b[part][word * 4 + 2] = bf16x2_to_f16x2(v.z);
            b[part][word * 4 + 3] = bf16x2_to_f16x2(v.w);
          }
        } else {
#pragma unroll
          for (int item = 0; item < 16; ++item) b[part][item] = 0u;
        }
      }
      for (int tile_index = 0; tile_index < my_tiles; ++tile_index) {
        copy_async_wait<kAhead - 1>();       // this lane's copies of the oldest tile have landed
        const uint32_t tile_base = lane_slot + ring_tile * (CPW * kSlotBytes);
#pragma unroll
        for (int part = 0; part < CPW; ++part) {
          const uint32_t base = tile_base + part * kSlotBytes;
          // both scale bytes of a row (K blocks 2 quad, 2 quad + 1 of the chunk) in one load
          const uint32_t scale_address = base + scale_slot + (quad & 1) * 2;
          const uint32_t scales_low = decode_scales(load_shared_u16(scale_address));
          const uint32_t scales_high = decode_scales(load_shared_u16(scale_address + 128));
          const uint4 packed_low = load_shared_16(base);
          const uint4 packed_high = load_shared_16(base + 512);
          const uint32_t multiplier_low[2] = {prmt(scales_low, scales_low, 0x1010u),
                                              prmt(scales_low, scales_low, 0x3232u)};
          const uint32_t multiplier_high[2] = {prmt(scales_high, scales_high, 0x1010u),
                                               prmt(scales_high, scales_high, 0x3232u)};
          const uint32_t words_low[4] = {packed_low.x, packed_low.y, packed_low.z, packed_low.w};
          const uint32_t words_high[4] = {packed_high.x, packed_high.y, packed_high.z, packed_high.w};
#pragma unroll
          for (int word = 0; word < 4; ++word) {
            // Eight codes of each row -> (w0,w1) (w2,w3) (w4,w5) (w6,w7), times the block scale:
            // exact in f16 (6 significant bits, magnitude within [2^-10, 2688]).
            uint32_t low[4], high[4];
            decode_e2m1x8(words_low[word], low);
            decode_e2m1x8(words_high[word], high);
            const uint32_t scale_low = multiplier_low[word >> 1];
            const uint32_t scale_high = multiplier_high[word >> 1];
            mma_f16_16x8x16(even, mul_f16x2(low[0], scale_low), mul_f16x2(high[0], scale_high),
                            mul_f16x2(low[1], scale_low), mul_f16x2(high[1], scale_high),
                            b[part][word * 4 + 0], b[part][word * 4 + 1]);
            mma_f16_16x8x16(odd, mul_f16x2(low[2], scale_low), mul_f16x2(high[2], scale_high),
                            mul_f16x2(low[3], scale_low), mul_f16x2(high[3], scale_high),
                            b[part][word * 4 + 2], b[part][word * 4 + 3]);
          }
        }
        // The tile's bytes are in registers: refill its slots with the tile kAhead further on (one
        // group per tile, empty at the end, keeps the wait above counting right).
        if (fetched < total_tiles) {
          fetch(ahead_pass, ahead_tile, ring_tile);
          ++fetched;
          if (++ahead_tile == my_tiles) {
            ahead_tile = 0;
            ++ahead_pass;
          }
        }
        copy_async_commit();
        ring_tile = ring_tile + 1 == kAhead ? 0 : ring_tile + 1;
        // The tile's share of this pass is complete in this warp: rows (group, group + 8) x
        // tokens (2 quad, 2 quad + 1).
        // (Once a wait has run out, `abort` is raised and this lane skips every later wait: the
        // loops run to their end with meaningless sums and the launch reports the failure.)
        if (alive) alive = ptx::mbarrier_wait(&sums_empty[buffer], buffer_phase ^ 1u, abort);
        __syncwarp();
        float* sums = reinterpret_cast<float*>(shared + SharedLayout::kSums + buffer * kSumBufferBytes) +
                      warp * kTileOutputs;
        *reinterpret_cast<float2*>(sums + group * 8 + 2 * quad) = make_float2(even[0] + odd[0], even[1] + odd[1]);
        *reinterpret_cast<float2*>(sums + (group + 8) * 8 + 2 * quad) =
            make_float2(even[2] + odd[2], even[3] + odd[3]);
#pragma unroll
        for (int item = 0; item < 4; ++item) even[item] = odd[item] = 0.0f;
        __syncwarp();
        if (lane == 0) ptx::mbarrier_arrive(&sums_full[buffer]);
        if (++buffer == kSumBuffers) {
          buffer = 0;
          buffer_phase ^= 1u;
        }
      }
    }
    copy_async_wait<0>();      // nothing of this CTA is in flight when it leaves
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort != 0u) *status = 1u;
}

using Kernel = void (*)(const uint8_t*, const uint8_t*, const void*, const uint8_t*, __nv_bfloat16*, int,
                        int, int, int, int, float, uint32_t*);

Kernel kernel_for(int chunks_per_warp, bool fp4_input) {
  switch (chunks_per_warp) {
    case 1: return fp4_input ? nvfp4_stream_kernel<1, true> : nvfp4_stream_kernel<1, false>;
    case 2: return fp4_input ? nvfp4_stream_kernel<2, true> : nvfp4_stream_kernel<2, false>;
    default: return fp4_input ? nvfp4_stream_kernel<3, true> : nvfp4_stream_kernel<3, false>;
  }
}

// K = 2048 * chunks_per_warp * passes with 1..3 chunks per warp; as few passes as possible.
static bool split_k(int k, int* chunks_per_warp, int* passes) {
  if (k <= 0 || k % kStageK != 0) return false;
  const int stages = k / kStageK;
  int first = kMaxChunksPerWarp;
  if (const char* forced = std::getenv("MIRCUDA_B200_NVFP4_CHUNKS")) {     // tuning knob
    const int value = std::atoi(forced);
    if (value >= 1 && value <= kMaxChunksPerWarp) first = value;
  }
  for (int chunks = first; chunks >= 1; --chunks) {
    if (stages % chunks == 0) {
      *chunks_per_warp = chunks;
      *passes = stages / chunks;
      return true;
    }
  }
  return false;
}

bool eligible(int n, int k) {
  int chunks = 0, passes = 0;
  return n > 0 && n % 128 == 0 && split_k(k, &chunks, &passes);
}

int prepare(Config* config, int n, int k) {
  if (!eligible(n, k)) return -1;
  split_k(k, &config->chunks_per_warp, &config->passes);
  int status = 0;
  for (int fp4_input = 0; fp4_input < 2 && status == 0; ++fp4_input) {
    status = static_cast<int>(cudaFuncSetAttribute(kernel_for(config->chunks_per_warp, fp4_input != 0),
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   SharedLayout::kBytes));
  }
  if (status != 0) return status;
  int device = 0, sm_count = 0;
  status = static_cast<int>(cudaGetDevice(&device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  }
  if (status != 0) return status;
  const int tiles = n / kTileRows;
  config->ctas = sm_count < tiles ? sm_count : tiles;
  // Several passes keep every tile's running sums in shared memory.
  if (config->passes > 1 && (tiles + config->ctas - 1) / config->ctas > kMaxTilesPerCta) return -1;
  return 0;
}

int launch(Config* config, cudaStream_t stream, bool overlap_launches, const void* input,
           const void* input_scales, const void* weight, const void* weight_scales, void* output, int m,
           int n, int k, float global_scale, uint32_t* status) {
  cudaLaunchConfig_t launch_config = {};
  launch_config.gridDim = dim3(config->ctas, 1, 1);
  launch_config.blockDim = dim3(kThreads, 1, 1);
  launch_config.dynamicSmemBytes = SharedLayout::kBytes;
  launch_config.stream = stream;
  cudaLaunchAttribute attributes[1] = {};
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  launch_config.attrs = attributes;
  launch_config.numAttrs = overlap_launches ? 1 : 0;
  return static_cast<int>(cudaLaunchKernelEx(
      &launch_config, kernel_for(config->chunks_per_warp, input_scales != nullptr),
      static_cast<const uint8_t*>(weight), static_cast<const uint8_t*>(weight_scales), input,
      static_cast<const uint8_t*>(input_scales), static_cast<__nv_bfloat16*>(output), m, n, k,
      n / kTileRows, config->passes, global_scale, status));
}

}  // namespace nvfp4_stream
}  // namespace mircuda_b200
