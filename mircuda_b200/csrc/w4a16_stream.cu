// int4-g128 W4A16 decode (M <= 16), streaming kernel:
//   y[m, n] = f16(sum_k x[m, k] * (q[n, k] - 8) * s[n, k / 128])
// The machine of nvfp4_stream.cu (one persistent CTA per SM over 16-row tiles, sixteen consumer
// warps that each own one 128-element K chunk of every 2048-element stage and keep their
// activation fragments in registers, lane-private cp.async rings instead of a producer, a
// reducer warp, passes over K with running sums in shared memory) around the int4 arithmetic
// of w4a16_int4.cu: a nibble OR-ed into the mantissa of 1024.0 is 1024 + q, one exact packed
// subtract (or multiply-add for the high nibbles) gives q - 8; a warp's chunk is exactly one
// scale group, so the f16 scale multiplies the chunk's fp32 sums once, after the MMAs.
// A tile is 16 consecutive weight rows; with more than 8 tokens every A fragment feeds two MMAs
// (two groups of 8 tokens).
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>

#include "ptx.cuh"
#include "w4a16_stream.hpp"

namespace mircuda_b200 {
namespace w4a16_stream {

constexpr int kConsumerWarps = 16;
constexpr int kReducerWarp = kConsumerWarps;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileRows = 16;
constexpr int kStageChunks = kConsumerWarps;
constexpr int kStageK = kStageChunks * 128;                  // 2048
constexpr int kSlotWeightBytes = 2 * 32 * 16;                // two rows x 32 lanes x 16 bytes
constexpr int kSlotScaleBytes = 2 * 32 * 4;                  // two rows x 32 lanes x one 4-byte word
constexpr int kSlotBytes = kSlotWeightBytes + kSlotScaleBytes;
constexpr int kSumBuffers = 4;
constexpr int kMaxChunksPerWarp = 2;
constexpr int kMaxTilesPerCta = 32;                          // running sums kept across passes

// TG token groups of 8; CPW chunks per warp and tile.
template <int TG, int CPW>
struct Shape {
  static constexpr int kAheadTiles = (TG == 2 ? 6 : 8) / CPW;       // tiles in flight per warp
  static constexpr int kSlots = kAheadTiles * CPW;
  static constexpr int kWarpRingBytes = kSlots * kSlotBytes;
  static constexpr int kTileOutputs = kTileRows * 8 * TG;
  static constexpr int kSumBufferBytes = kConsumerWarps * kTileOutputs * 4;
  static constexpr int kRings = 0;
  static constexpr int kSums = kRings + kConsumerWarps * kWarpRingBytes;
  static constexpr int kRunning = kSums + kSumBuffers * kSumBufferBytes;
  static constexpr int kBarriers = kRunning + kMaxTilesPerCta * kTileOutputs * 4;
  static constexpr int kAbort = kBarriers + 2 * kSumBuffers * 8;
  static constexpr int kBytes = kAbort + 16;
  static_assert(kBytes <= 232448, "fits the shared memory of one SM");
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t bits) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(d) : "r"(a), "r"(mask), "r"(bits));   // (a & b) | c
  return d;
}

__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

// Eight codes of one u32 (k0..k7, k0 lowest) -> (k0,k4) (k1,k5) (k2,k6) (k3,k7) as q - 8 in
// f16x2, exactly: 1024 + q minus 1032, and (1024 + 16 q) / 16 minus 72. The shift by one byte
// is an integer multiply-high: it runs on the FMA pipe, the logic pipe is the scarce one.
__device__ __forceinline__ void dequantize8(uint32_t codes, uint32_t (&out)[4]) {
  const uint32_t shifted = __umulhi(codes, 1u << 24);
  out[0] = sub_f16x2(lop3_and_or(codes, 0x000f000fu, 0x64006400u), 0x64086408u);
  out[1] = fma_f16x2(lop3_and_or(codes, 0x00f000f0u, 0x64006400u), 0x2c002c00u, 0xd480d480u);
  out[2] = sub_f16x2(lop3_and_or(shifted, 0x000f000fu, 0x64006400u), 0x64086408u);
  out[3] = fma_f16x2(lop3_and_or(shifted, 0x00f000f0u, 0x64006400u), 0x2c002c00u, 0xd480d480u);
}

// D = A * B (+ C): the first MMA of a chunk starts from zero accumulators.
__device__ __forceinline__ void mma_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ void mma_next(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
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

__device__ __forceinline__ void mbarrier_arrive_after(uint32_t barrier, uint32_t token) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(barrier), "r"(token) : "memory");
}

template <int TG, int CPW>
__global__ void __launch_bounds__(kThreads, 1)
w4a16_stream_kernel(const uint8_t* __restrict__ weight, const __half* __restrict__ scales,
                    const __half* __restrict__ input, __half* __restrict__ output, int m, int n, int k,
                    int tiles, int passes, uint32_t* __restrict__ status) {
  using S = Shape<TG, CPW>;
  extern __shared__ __align__(16) uint8_t shared[];
  const uint32_t shared_base = ptx::smem_address(shared);
  uint64_t* sums_full = reinterpret_cast<uint64_t*>(shared + S::kBarriers);
  uint64_t* sums_empty = sums_full + kSumBuffers;
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(shared + S::kAbort);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grid = static_cast<int>(gridDim.x);
  const int cta = static_cast<int>(blockIdx.x);
  const int my_tiles = cta < tiles ? (tiles - cta + grid - 1) / grid : 0;

  // Programmatic dependent launch (a no-op unless the launch asked for it): weights and scales
  // are taken to be constant and are fetched at once; activations are read and outputs written
  // only after the previous kernel of the stream has completed.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
        float4 total[TG];
#pragma unroll
        for (int tokens = 0; tokens < TG; ++tokens) {
          const uint32_t source = shared_base + S::kSums + buffer * S::kSumBufferBytes + tokens * 512 + lane * 16;
          total[tokens] = load_shared_float4(source);
#pragma unroll
          for (int other = 1; other < kConsumerWarps; ++other) {
            const float4 v = load_shared_float4(source + other * S::kTileOutputs * 4);
            total[tokens].x += v.x;
            total[tokens].y += v.y;
            total[tokens].z += v.z;
            total[tokens].w += v.w;
          }
        }
        __syncwarp();
        if (lane == 0) {
          mbarrier_arrive_after(ptx::smem_address(&sums_empty[buffer]), __float_as_uint(total[TG - 1].x));
        }
        if (++buffer == kSumBuffers) {
          buffer = 0;
          buffer_phase ^= 1u;
        }
        bool finish = true;
        if (passes > 1) {
#pragma unroll
          for (int tokens = 0; tokens < TG; ++tokens) {
            const uint32_t running = shared_base + S::kRunning + tile_index * S::kTileOutputs * 4 + tokens * 512 + lane * 16;
            if (pass > 0) {
              const float4 v = load_shared_float4(running);
              total[tokens].x += v.x;
              total[tokens].y += v.y;
              total[tokens].z += v.z;
              total[tokens].w += v.w;
            }
            if (pass + 1 < passes) store_shared_float4(running, total[tokens]);
          }
          finish = pass + 1 == passes;
        }
        if (!finish) continue;
        // lane -> row lane / 2 of the tile, tokens 8 * group + 4 * (lane % 2) .. + 3
        const int row = (cta + tile_index * grid) * kTileRows + (lane >> 1);
#pragma unroll
        for (int tokens = 0; tokens < TG; ++tokens) {
          const int token = tokens * 8 + (lane & 1) * 4;
          const float values[4] = {total[tokens].x, total[tokens].y, total[tokens].z, total[tokens].w};
#pragma unroll
          for (int item = 0; item < 4; ++item) {
            if (token + item < m) output[static_cast<size_t>(token + item) * n + row] = __float2half_rn(values[item]);
          }
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- consumers
    const int group = lane >> 2;
    const int quad = lane & 3;
    const int groups_k = k / 128;
    const size_t row_bytes = static_cast<size_t>(k) / 2;
    const uint32_t ring = shared_base + S::kRings + warp * S::kWarpRingBytes;
    const int total_tiles = passes * my_tiles;
    constexpr int kAhead = S::kAheadTiles;
    // MMA rows `group` and `group + 8` are rows group and group + 8 of the tile; this lane's 16
    // bytes of a row are K elements 32 quad .. + 31 of the warp's chunk.
    const uint8_t* const lane_weight = weight + static_cast<size_t>(group) * row_bytes + warp * 64 + quad * 16;
    const uint32_t lane_slot = ring + lane * 16;
    const uint32_t scale_slot = kSlotWeightBytes - lane * 12;   // this lane's scale words, relative to lane_slot

    // Fetches all CPW chunks of one tile of one pass into the ring slots of `ring_tile`. The f16
    // scale of (row, chunk) arrives inside the aligned 4-byte word that holds it.
    auto fetch = [&](int pass, int tile_index, int ring_tile) {
      const int first_row = (cta + tile_index * grid) * kTileRows;
      const int chunk = pass * (CPW * kStageChunks) + warp;
      const uint8_t* low = lane_weight + static_cast<size_t>(first_row) * row_bytes +
                           pass * (CPW * kStageChunks * 64);
      uint32_t destination = lane_slot + ring_tile * (CPW * kSlotBytes);
      size_t scale_low = static_cast<size_t>(first_row + group) * groups_k + chunk;
#pragma unroll
      for (int part = 0; part < CPW; ++part) {
        copy_async_16(destination, low);
        copy_async_16(destination + 512, low + 8 * row_bytes);
        const size_t scale_high = scale_low + static_cast<size_t>(8) * groups_k;
        copy_async_4(destination + scale_slot, scales + (scale_low & ~static_cast<size_t>(1)));
        copy_async_4(destination + scale_slot + 128, scales + (scale_high & ~static_cast<size_t>(1)));
        destination += kSlotBytes;
        low += kStageChunks * 64;
        scale_low += kStageChunks;
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

    float total[TG][4];
#pragma unroll
    for (int tokens = 0; tokens < TG; ++tokens) {
#pragma unroll
      for (int item = 0; item < 4; ++item) total[tokens][item] = 0.0f;
    }
    uint32_t ring_tile = 0, buffer = 0, buffer_phase = 0;
    bool alive = true;
    for (int pass = 0; pass < passes; ++pass) {
      // B fragments of this pass: tokens `group` and `group + 8`, this lane's 32 K-elements of the
      // warp's chunk of every stage, paired (k, k + 4) as the dequantiser pairs the weights.
      uint32_t b[CPW][TG][16];
#pragma unroll
      for (int part = 0; part < CPW; ++part) {
        const int element = ((pass * CPW + part) * kStageChunks + warp) * 128 + quad * 32;
#pragma unroll
        for (int tokens = 0; tokens < TG; ++tokens) {
          const int token = tokens * 8 + group;
          if (token < m) {
            const uint4* source = reinterpret_cast<const uint4*>(input + static_cast<size_t>(token) * k + element);
#pragma unroll
            for (int word = 0; word < 4; ++word) {
              const uint4 v = __ldg(source + word);       // x0..x7 as (x0,x1) (x2,x3) (x4,x5) (x6,x7)
              b[part][tokens][word * 4 + 0] = prmt(v.x, v.z, 0x5410u);   // (x0, x4)
              b[part][tokens][word * 4 + 1] = prmt(v.x, v.z, 0x7632u);   // (x1, x5)
              b[part][tokens][word * 4 + 2] = prmt(v.y, v.w, 0x5410u);   // (x2, x6)
              b[part][tokens][word * 4 + 3] = prmt(v.y, v.w, 0x7632u);   // (x3, x7)
            }
          } else {
#pragma unroll
            for (int item = 0; item < 16; ++item) b[part][tokens][item] = 0u;
          }
        }
      }
      for (int tile_index = 0; tile_index < my_tiles; ++tile_index) {
        copy_async_wait<kAhead - 1>();
        const uint32_t tile_base = lane_slot + ring_tile * (CPW * kSlotBytes);
        const int first_row = (cta + tile_index * grid) * kTileRows;
#pragma unroll
        for (int part = 0; part < CPW; ++part) {
          const uint32_t base = tile_base + part * kSlotBytes;
          // which half of the fetched word holds the scale: parity of its element index
          const int chunk = (pass * CPW + part) * kStageChunks + warp;
          const uint32_t low_half = static_cast<uint32_t>((static_cast<size_t>(first_row + group) * groups_k + chunk) & 1u);
          const uint32_t high_half = static_cast<uint32_t>((static_cast<size_t>(first_row + group + 8) * groups_k + chunk) & 1u);
          const float scale_low = __half2float(__ushort_as_half(
              static_cast<unsigned short>(load_shared_u16(base + scale_slot + low_half * 2))));
          const float scale_high = __half2float(__ushort_as_half(
              static_cast<unsigned short>(load_shared_u16(base + scale_slot + 128 + high_half * 2))));
          const uint4 packed_low = load_shared_16(base);
          const uint4 packed_high = load_shared_16(base + 512);
          const uint32_t words_low[4] = {packed_low.x, packed_low.y, packed_low.z, packed_low.w};
          const uint32_t words_high[4] = {packed_high.x, packed_high.y, packed_high.z, packed_high.w};
          float even[TG][4], odd[TG][4];
#pragma unroll
          for (int word = 0; word < 4; ++word) {
            uint32_t low[4], high[4];
            dequantize8(words_low[word], low);
            dequantize8(words_high[word], high);
#pragma unroll
            for (int tokens = 0; tokens < TG; ++tokens) {
              if (word == 0) {
                mma_first(even[tokens], low[0], high[0], low[1], high[1], b[part][tokens][0], b[part][tokens][1]);
                mma_first(odd[tokens], low[2], high[2], low[3], high[3], b[part][tokens][2], b[part][tokens][3]);
              } else {
                mma_next(even[tokens], low[0], high[0], low[1], high[1], b[part][tokens][word * 4 + 0],
                         b[part][tokens][word * 4 + 1]);
                mma_next(odd[tokens], low[2], high[2], low[3], high[3], b[part][tokens][word * 4 + 2],
                         b[part][tokens][word * 4 + 3]);
              }
            }
          }
          // the chunk is one scale group of each row: scale its sums once, in fp32
#pragma unroll
          for (int tokens = 0; tokens < TG; ++tokens) {
            total[tokens][0] = fmaf(scale_low, even[tokens][0] + odd[tokens][0], total[tokens][0]);
            total[tokens][1] = fmaf(scale_low, even[tokens][1] + odd[tokens][1], total[tokens][1]);
            total[tokens][2] = fmaf(scale_high, even[tokens][2] + odd[tokens][2], total[tokens][2]);
            total[tokens][3] = fmaf(scale_high, even[tokens][3] + odd[tokens][3], total[tokens][3]);
          }
        }
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
        // rows (group, group + 8) x tokens (2 quad, 2 quad + 1) of every token group
        if (alive) alive = ptx::mbarrier_wait(&sums_empty[buffer], buffer_phase ^ 1u, abort);
        __syncwarp();
        float* sums = reinterpret_cast<float*>(shared + S::kSums + buffer * S::kSumBufferBytes) +
                      warp * S::kTileOutputs;
#pragma unroll
        for (int tokens = 0; tokens < TG; ++tokens) {
          *reinterpret_cast<float2*>(sums + tokens * 128 + group * 8 + 2 * quad) =
              make_float2(total[tokens][0], total[tokens][1]);
          *reinterpret_cast<float2*>(sums + tokens * 128 + (group + 8) * 8 + 2 * quad) =
              make_float2(total[tokens][2], total[tokens][3]);
#pragma unroll
          for (int item = 0; item < 4; ++item) total[tokens][item] = 0.0f;
        }
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

using Kernel = void (*)(const uint8_t*, const __half*, const __half*, __half*, int, int, int, int, int, uint32_t*);

static Kernel kernel_for(int token_groups, int chunks_per_warp) {
  if (token_groups == 2) return w4a16_stream_kernel<2, 1>;
  return chunks_per_warp == 2 ? w4a16_stream_kernel<1, 2> : w4a16_stream_kernel<1, 1>;
}

static int shared_bytes(int token_groups, int chunks_per_warp) {
  if (token_groups == 2) return Shape<2, 1>::kBytes;
  return chunks_per_warp == 2 ? Shape<1, 2>::kBytes : Shape<1, 1>::kBytes;
}

int prepare(Config* config, int m, int n, int k) {
  if (m <= 0 || m > 16 || n <= 0 || n % kTileRows != 0 || k <= 0 || k % kStageK != 0) return -1;
  const int stages = k / kStageK;
  config->token_groups = m <= 8 ? 1 : 2;
  // two chunks per warp halve the passes; with two token groups the fragments of one chunk
  // already take 32 registers
  config->chunks_per_warp = (config->token_groups == 1 && stages % 2 == 0) ? 2 : 1;
  config->passes = stages / config->chunks_per_warp;
  // With two token groups and many passes (K = 14336: seven) the ring kernel measured faster
  // (19.6 against 20.6 us at N = 4096, M = 16): the running sums of 16 tokens are read and
  // written once per pass.
  if (config->token_groups == 2 && config->passes > 2) return -1;
  int device = 0, sm_count = 0;
  int status = static_cast<int>(cudaGetDevice(&device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  }
  if (status != 0) return status;
  const int tiles = n / kTileRows;
  config->ctas = sm_count < tiles ? sm_count : tiles;
  if (config->passes > 1 && (tiles + config->ctas - 1) / config->ctas > kMaxTilesPerCta) return -1;
  return static_cast<int>(cudaFuncSetAttribute(kernel_for(config->token_groups, config->chunks_per_warp),
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               shared_bytes(config->token_groups, config->chunks_per_warp)));
}

int launch(const Config* config, cudaStream_t stream, bool overlap_launches, const void* input,
           const void* weight, const void* scales, void* output, int m, int n, int k, uint32_t* status) {
  cudaLaunchConfig_t launch_config = {};
  launch_config.gridDim = dim3(config->ctas, 1, 1);
  launch_config.blockDim = dim3(kThreads, 1, 1);
  launch_config.dynamicSmemBytes = shared_bytes(config->token_groups, config->chunks_per_warp);
  launch_config.stream = stream;
  cudaLaunchAttribute attributes[1] = {};
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  launch_config.attrs = attributes;
  launch_config.numAttrs = overlap_launches ? 1 : 0;
  return static_cast<int>(cudaLaunchKernelEx(
      &launch_config, kernel_for(config->token_groups, config->chunks_per_warp),
      static_cast<const uint8_t*>(weight), static_cast<const __half*>(scales),
      static_cast<const __half*>(input), static_cast<__half*>(output), m, n, k, n / kTileRows,
      config->passes, status));
}

}  // namespace w4a16_stream
}  // namespace mircuda_b200
