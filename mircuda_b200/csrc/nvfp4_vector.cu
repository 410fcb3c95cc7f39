// bf16-activation x NVFP4-weight skinny GEMM for decode, M <= 8:
//   y[m, n] = bf16(global * sum_k x[m, k] * e2m1(W[n, k]) * ue4m3(s[n, k / 16]))
// Weights [N, K/2] (two codes per byte, even k low) and swizzled UE4M3 scales use the same
// layouts as the FP4 x FP4 GEMV. This entry point has no counterpart in the reference's C
// ABI; the reference serves this shape through its Marlin NVFP4 dense path, whose numerics
// (exact weight * scale products, fp32 accumulation, global scale before the bf16 round)
// it follows.
//
// Three kernels sit behind the plan. Shapes with n % 128 == 0 and k % 2048 == 0 run on the
// streaming kernel of nvfp4_stream.cu (MIRCUDA_B200_NVFP4_VECTOR=stream, the default there); the
// two kernels of this file serve every other shape: `nvfp4_direct_kernel` (global loads through
// a register pipeline; the default among the two) and `nvfp4_vector_kernel` (the TMA-fed ring
// described next; MIRCUDA_B200_NVFP4_VECTOR=ring).
//
// The op streams 0.5625*N*K bytes once and is bound by HBM, so the kernel is built around
// keeping bytes in flight rather than around arithmetic:
//  * a CTA owns one 128-row scale tile and a contiguous part of K; a producer warp streams
//    that part in stages of 512 K-elements (a [128 x 256 B] weight box by TMA plus the eight
//    512-byte scale atoms by one bulk copy) through a two-stage shared-memory ring, and two
//    CTAs fit on an SM (four stages, 144 KB, in flight per SM; 256-element stages in a
//    four-deep ring measured 20 % slower);
//  * eight consumer warps turn E2M1 codes into f16x2 with the hardware conversion (one
//    instruction per two weights; an earlier bit-placement version spent four instructions
//    per weight and was bound by the integer pipe), multiply by the block scale with one
//    exact packed f16 multiply and feed mma.sync.m16n8k16 with the weights on the 16-row side
//    and the tokens on the 8-wide side, so the cost does not grow with M; activations are
//    tiny, come straight from L2 into registers and are converted bf16 -> f16 there (exact
//    for magnitudes in [2^-14, 65504], saturating above);
//  * when N alone does not give enough CTAs, K is cut into 2, 4 or 8 parts that form a
//    thread-block cluster; the parts' partial sums meet in the first CTA's shared memory
//    (distributed shared memory, one cluster barrier) instead of in global memory.
// Every mbarrier wait is bounded; the cluster barrier is reached on every path.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>

#include "fp4_codec.cuh"
#include "nvfp4_stream.hpp"
#include "ptx.cuh"
#include "ptx_pair.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace nvfp4_vector {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;   // + one producer warp
constexpr int kTileRows = 128;
constexpr int kStageK = 512;                          // K-elements per stage
constexpr int kStageWeightBytes = kTileRows * kStageK / 2;   // 32 KB
constexpr int kStageScaleBytes = (kStageK / 64) * 512;       // 8 atoms = 4 KB
constexpr int kStages = 2;
constexpr int kWarpsK = kStageK / 128;                // consumer warps side by side along K
constexpr int kRowGroups = kConsumerWarps / kWarpsK;  // ... and along the rows
constexpr int kRowsPerWarp = kTileRows / kRowGroups;
constexpr int kSteps = kRowsPerWarp / 16;             // 16-row MMA steps per warp and stage
constexpr int kMaxTokens = 8;
constexpr int kMaxParts = 8;

struct Plan {
  int m, n, k;
  int parts;                 // K parts = cluster size along y
  bool overlap_launches;     // programmatic dependent launch (MIRCUDA_B200_OVERLAP_LAUNCHES=1)
  bool direct;               // the kernel without the shared-memory ring
  bool stream_kernel;        // the persistent streaming kernel of nvfp4_stream.cu
  nvfp4_stream::Config stream_config;
  int device;
  cudaStream_t stream;
  uint32_t* status;          // pinned; set when a bounded wait ran out
  const void* cached_weight;
  CUtensorMap weight_map;    // [N, K/2] bytes, box 256 B x 128 rows, no swizzle
};

struct SharedLayout {
  static constexpr int kWeights = 0;
  static constexpr int kSums = 0;      // [kWarpsK][128][8] f32, reuses the ring after the main loop
  static constexpr int kScales = kStages * kStageWeightBytes;
  static constexpr int kParts = kScales + kStages * kStageScaleBytes;            // [8][128][8] f32
  static constexpr int kBarriers = kParts + kMaxParts * kTileRows * kMaxTokens * 4;
  static constexpr int kBytes = kBarriers + 2 * kStages * 8 + 16 + 1024;         // + alignment slack
  static_assert(kWarpsK * kTileRows * kMaxTokens * 4 <= kStages * kStageWeightBytes, "sums fit the ring");
  static_assert(2 * kBytes <= 232448, "two CTAs per SM");
};

// Eight E2M1 codes (one u32, even k in the low nibble of each byte) -> four f16x2 in K order,
// with the sm_100a conversion instruction: one instruction per two weights.
__device__ __forceinline__ void decode_e2m1x8_bits(uint32_t codes, uint32_t (&out)[4]) {
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

// Two E4M3 codes (low 16 bits) -> f16x2, exact.
__device__ __forceinline__ uint32_t decode_e4m3x2(uint32_t two_codes) {
  uint32_t pair;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(static_cast<uint16_t>(two_codes)));
  return pair;
}

__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Two bf16 -> two f16 (round to nearest, saturating at +-65504). Exact for every value whose
// magnitude lies in [2^-14, 65504]; smaller ones keep an absolute error below 2^-25.
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

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

__global__ void __launch_bounds__(kThreads)
nvfp4_vector_kernel(const __grid_constant__ CUtensorMap weight_map,
                    const __nv_bfloat16* __restrict__ input,
                    const uint8_t* __restrict__ weight_scales,
                    __nv_bfloat16* __restrict__ output, int m, int n, int k, int parts,
                    float global_scale, uint32_t* __restrict__ status) {
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_weights = shared + SharedLayout::kWeights;
  uint8_t* shared_scales = shared + SharedLayout::kScales;
  float* shared_sums = reinterpret_cast<float*>(shared + SharedLayout::kSums);
  float* shared_parts = reinterpret_cast<float*>(shared + SharedLayout::kParts);
  uint64_t* full = reinterpret_cast<uint64_t*>(shared + SharedLayout::kBarriers);
  uint64_t* empty = full + kStages;
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(empty + kStages);

  const int row_tile = blockIdx.x;
  const int part = blockIdx.y;                       // == rank inside the cluster
  const int stages_total = (k + kStageK - 1) / kStageK;
  const int stages_per_part = (stages_total + parts - 1) / parts;
  const int first_stage = part * stages_per_part;
  const int my_stages = max(0, min(stages_per_part, stages_total - first_stage));
  const int atoms_k = k / 64;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int stage = 0; stage < kStages; ++stage) {
      ptx::mbarrier_init(&full[stage], 1);
      ptx::mbarrier_init(&empty[stage], kConsumerWarps);
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&weight_map);
  }
  __syncthreads();
  // Programmatic dependent launch (a no-op unless the launch asked for it): the next kernel
  // in the stream may start as soon as every CTA of this one has got here, and this kernel
  // may have started before the previous one finished. Weights and their scales are taken to
  // be constant, so the producer streams them at once; every thread waits for the previous
  // kernel to complete before it first reads activations or writes outputs.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == kConsumerWarps) {
    // --------------------------------------------------------------------- producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      for (int index = 0; index < my_stages; ++index) {
        if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) break;
        const int global_stage = first_stage + index;
        const int atoms_here = min(kStageK / 64, atoms_k - global_stage * (kStageK / 64));
        ptx::mbarrier_arrive_expect_tx(&full[stage], kStageWeightBytes + atoms_here * 512);
        ptx::tma_load_2d(shared_weights + stage * kStageWeightBytes, &weight_map, &full[stage],
                         global_stage * (kStageK / 2), row_tile * kTileRows);
        ptx::bulk_load(shared_scales + stage * kStageScaleBytes,
                       weight_scales + (static_cast<size_t>(row_tile) * atoms_k +
                                        static_cast<size_t>(global_stage) * (kStageK / 64)) * 512,
                       atoms_here * 512, &full[stage]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (*abort != 0u) {
        for (int spin = 0; spin < 256; ++spin) __nanosleep(1000);
      }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
  } else {
    // -------------------------------------------------------------------- consumers
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int group = lane >> 2;                     // weight row inside a 16-row step / token
    const int quad = lane & 3;
    const int warp_k = warp % kWarpsK;               // 128-element K sub-range of the stage
    const int warp_rows = warp / kWarpsK;            // kRowsPerWarp rows of the tile
    const int chunk = warp_k * 4 + quad;             // this thread's 32-element chunk
    float accumulator[kSteps][4];
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
#pragma unroll
      for (int item = 0; item < 4; ++item) accumulator[step][item] = 0.0f;
    }
    uint32_t stage = 0, phase = 0;
    for (int index = 0; index < my_stages; ++index) {
      const int element = (first_stage + index) * kStageK + chunk * 32;
      // B fragments first (from L2; independent of the stage's arrival): token `group`,
      // 32 consecutive activations as f16x2 pairs in K order.
      uint32_t b[16];
      if (group < m && element < k) {
        const uint4* source = reinterpret_cast<const uint4*>(input + static_cast<size_t>(group) * k + element);
#pragma unroll
        for (int word = 0; word < 4; ++word) {
          const uint4 v = __ldg(source + word);       // x0..x7 as (x0,x1) (x2,x3) (x4,x5) (x6,x7)
          b[word * 4 + 0] = bf16x2_to_f16x2(v.x);
          b[word * 4 + 1] = bf16x2_to_f16x2(v.y);
          b[word * 4 + 2] = bf16x2_to_f16x2(v.z);
          b[word * 4 + 3] = bf16x2_to_f16x2(v.w);
        }
      } else {
#pragma unroll
        for (int item = 0; item < 16; ++item) b[item] = 0u;
      }
      if (!ptx::mbarrier_wait(&full[stage], phase, abort)) break;
      const uint8_t* weights = shared_weights + stage * kStageWeightBytes;
      const uint8_t* scales = shared_scales + stage * kStageScaleBytes;
      const bool active = element < k;
#pragma unroll
      for (int step = 0; step < kSteps; ++step) {
        const int row_low = warp_rows * kRowsPerWarp + step * 16 + group;
        const int row_high = row_low + 8;
        const uint4 packed_low = *reinterpret_cast<const uint4*>(weights + row_low * (kStageK / 2) + chunk * 16);
        const uint4 packed_high = *reinterpret_cast<const uint4*>(weights + row_high * (kStageK / 2) + chunk * 16);
        const uint32_t two_low = *reinterpret_cast<const uint16_t*>(
            scales + (chunk >> 1) * 512 + (row_low & 31) * 16 + (row_low >> 5) * 4 + (chunk & 1) * 2);
        const uint32_t two_high = *reinterpret_cast<const uint16_t*>(
            scales + (chunk >> 1) * 512 + (row_high & 31) * 16 + (row_high >> 5) * 4 + (chunk & 1) * 2);
        // Both block scales of the chunk in one conversion (UE4M3 is exact in f16), then each
        // broadcast to both halves of a register.
        // A chunk past the end of K holds zero codes (TMA fill) but stale scale bytes: force
        // those scales to zero too. The MMAs themselves run in every lane (mma.sync needs the
        // whole warp converged).
        const uint32_t scale_mask = active ? 0x7f7fu : 0u;
        const uint32_t both_low = decode_e4m3x2(two_low & scale_mask);
        const uint32_t both_high = decode_e4m3x2(two_high & scale_mask);
        const uint32_t multiplier_low[2] = {prmt(both_low, both_low, 0x1010u), prmt(both_low, both_low, 0x3232u)};
        const uint32_t multiplier_high[2] = {prmt(both_high, both_high, 0x1010u),
                                             prmt(both_high, both_high, 0x3232u)};
        const uint32_t words_low[4] = {packed_low.x, packed_low.y, packed_low.z, packed_low.w};
        const uint32_t words_high[4] = {packed_high.x, packed_high.y, packed_high.z, packed_high.w};
#pragma unroll
        for (int word = 0; word < 4; ++word) {
          // Eight codes -> (w0,w1) (w2,w3) (w4,w5) (w6,w7) as f16x2, exact; times the block
          // scale, still exact in f16 (6 significant bits, magnitude within [2^-10, 2688]).
          uint32_t low[4], high[4];
          decode_e2m1x8_bits(words_low[word], low);
          decode_e2m1x8_bits(words_high[word], high);
          const uint32_t scale_low = multiplier_low[word >> 1];
          const uint32_t scale_high = multiplier_high[word >> 1];
#pragma unroll
          for (int pair = 0; pair < 2; ++pair) {
            mma_f16_16x8x16(accumulator[step], mul_f16x2(low[2 * pair], scale_low),
                            mul_f16x2(high[2 * pair], scale_high),
                            mul_f16x2(low[2 * pair + 1], scale_low),
                            mul_f16x2(high[2 * pair + 1], scale_high), b[word * 4 + 2 * pair],
                            b[word * 4 + 2 * pair + 1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbarrier_arrive(&empty[stage]);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    // All consumer warps are done with the ring before the sums overwrite it.
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
    // accumulator[step]: rows (group, group + 8) of the step x tokens (2*quad, 2*quad + 1)
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
      const int row = warp_rows * kRowsPerWarp + step * 16 + group;
      float* base = shared_sums + (warp_k * kTileRows + row) * kMaxTokens + 2 * quad;
      *reinterpret_cast<float2*>(base) = make_float2(accumulator[step][0], accumulator[step][1]);
      *reinterpret_cast<float2*>(base + 8 * kMaxTokens) =
          make_float2(accumulator[step][2], accumulator[step][3]);
    }
  }
  __syncthreads();

  // CTA partial [128 rows][8 tokens] = sum over the K sub-ranges; it goes to slot `part`
  // of the first CTA's `shared_parts` (its own shared memory when there is one part).
  const uint32_t slot_base = ptx::smem_address(shared_parts + part * kTileRows * kMaxTokens);
  const uint32_t remote_base = parts > 1 ? ptx::map_to_cta(slot_base, 0u) : slot_base;
  for (int index = threadIdx.x; index < kTileRows * kMaxTokens; index += kThreads) {
    float sum = shared_sums[index];
#pragma unroll
    for (int sub = 1; sub < kWarpsK; ++sub) sum += shared_sums[sub * kTileRows * kMaxTokens + index];
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_base + index * 4), "f"(sum) : "memory");
  }
  if (parts > 1) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  if (part == 0) {
    const float finish = global_scale;
    for (int index = threadIdx.x; index < kTileRows * kMaxTokens; index += kThreads) {
      const int row = row_tile * kTileRows + index / kMaxTokens;
      const int token = index % kMaxTokens;
      float total = 0.0f;
      for (int slot = 0; slot < parts; ++slot) total += shared_parts[slot * kTileRows * kMaxTokens + index];
      if (row < n && token < m) {
        output[static_cast<size_t>(token) * n + row] = __float2bfloat16_rn(total * finish);
      }
    }
  }
  if (threadIdx.x == 0 && *abort != 0u) *status = 1u;
}

// The same op without the shared-memory ring: every consumer warp loads its weights, scale
// bytes and activations straight from global memory through a register pipeline (the next
// half stage always in flight), eight warps and no producer, no mbarrier. The ring version
// pays for its machinery on every launch (barrier set-up, descriptor fetch, a producer round
// trip before the first byte); this one starts computing one memory latency after launch,
// which is what decides the 8-25 MB shapes. Work split, K parts as a cluster and the
// hand-over of partial sums are those of the kernel above.
constexpr int kDirectThreads = kConsumerWarps * 32;
constexpr int kDirectSharedBytes =
    (kWarpsK + kMaxParts) * kTileRows * kMaxTokens * 4;      // warps' sums, then the parts' sums

template <bool WHOLE_STAGES>   // k % 512 == 0: no chunk of a stage lies past the end of K
__global__ void __launch_bounds__(kDirectThreads, 2)
nvfp4_direct_kernel(const uint8_t* __restrict__ weight, const __nv_bfloat16* __restrict__ input,
                    const uint8_t* __restrict__ weight_scales, __nv_bfloat16* __restrict__ output,
                    int m, int n, int k, int parts, float global_scale) {
  extern __shared__ __align__(16) uint8_t direct_shared[];
  float* shared_sums = reinterpret_cast<float*>(direct_shared);
  float* shared_parts = shared_sums + kWarpsK * kTileRows * kMaxTokens;

  const int row_tile = blockIdx.x;
  const int part = blockIdx.y;                       // == rank inside the cluster
  const int stages_total = (k + kStageK - 1) / kStageK;
  const int stages_per_part = (stages_total + parts - 1) / parts;
  const int first_stage = part * stages_per_part;
  const int my_stages = max(0, min(stages_per_part, stages_total - first_stage));
  const int atoms_k = k / 64;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = lane >> 2;
  const int quad = lane & 3;
  const int warp_k = warp % kWarpsK;
  const int warp_rows = warp / kWarpsK;
  const int chunk = warp_k * 4 + quad;               // this thread's 32-element chunk of a stage
  const size_t row_bytes = static_cast<size_t>(k) / 2;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  float accumulator[kSteps][4];
#pragma unroll
  for (int step = 0; step < kSteps; ++step) {
#pragma unroll
    for (int item = 0; item < 4; ++item) accumulator[step][item] = 0.0f;
  }
  // Rows of this lane: warp_rows * 64 + step * 16 + group (+ 8). Rows past n read row n - 1
  // (their sums are never stored).
  const uint8_t* row_pointer[kSteps][2];
#pragma unroll
  for (int step = 0; step < kSteps; ++step) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = row_tile * kTileRows + warp_rows * kRowsPerWarp + step * 16 + group + half * 8;
      row_pointer[step][half] = weight + static_cast<size_t>(min(row, n - 1)) * row_bytes + chunk * 16;
    }
  }
  // Scale bytes: rows 32 apart share a 16-byte line of an atom, one 4-byte word per quarter;
  // steps s and s + 2 of this lane are such rows, so one 8-byte load serves both.
  // line[j][half]: rows (j * 16 + group + half * 8) mod 32, quarters 2 * warp_rows + {0, 1}.
  const uint8_t* scale_base = weight_scales + static_cast<size_t>(row_tile) * atoms_k * 512 + warp_rows * 8;

  // Software pipeline over half stages (two 16-row steps each): while one half is being
  // computed the next half's weights are in flight, and so are the next stage's scale words
  // and activations. A CTA's stages would otherwise run as a chain of load latencies.
  auto load_weights = [&](int stage, int half, uint4 (&words)[2][2]) {
    const bool active = WHOLE_STAGES || stage * kStageK + chunk * 32 < k;
#pragma unroll
    for (int step = 0; step < 2; ++step) {
#pragma unroll
      for (int row_half = 0; row_half < 2; ++row_half) {
        words[step][row_half] =
            active ? load_streaming_16(row_pointer[half * 2 + step][row_half] + static_cast<size_t>(stage) * (kStageK / 2))
                   : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  auto load_scales = [&](int stage, uint2 (&words)[2][2]) {
    const int element = stage * kStageK + chunk * 32;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int row_half = 0; row_half < 2; ++row_half) {
        const int line = j * 16 + group + row_half * 8;
        words[j][row_half] =
            (WHOLE_STAGES || element < k) ? __ldg(reinterpret_cast<const uint2*>(scale_base + static_cast<size_t>(element / 64) * 512 + line * 16))
                        : make_uint2(0u, 0u);
      }
    }
  };
  auto load_tokens = [&](int stage, uint4 (&words)[4]) {
    const int element = stage * kStageK + chunk * 32;
    const bool has_token = group < m && (WHOLE_STAGES || element < k);
#pragma unroll
    for (int word = 0; word < 4; ++word) {
      words[word] = has_token ? __ldg(reinterpret_cast<const uint4*>(input + static_cast<size_t>(group) * k + element) + word)
                              : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  // Two steps (rows step * 16 + group, + 8) of one half: step = half * 2 + {0, 1}; their scale
  // words are line j = step % 2, component half (x for steps 0 and 1, y for steps 2 and 3).
  auto compute = [&](int half, const uint4 (&weights)[2][2], const uint2 (&scale_words)[2][2],
                     const uint32_t (&b)[16]) {
#pragma unroll
    for (int local = 0; local < 2; ++local) {
      const int step = half * 2 + local;
      const uint2 pair_low = scale_words[local][0];
      const uint2 pair_high = scale_words[local][1];
      const uint32_t word_low = half ? pair_low.y : pair_low.x;
      const uint32_t word_high = half ? pair_high.y : pair_high.x;
      const uint32_t both_low = decode_e4m3x2((word_low >> ((chunk & 1) * 16)) & 0x7f7fu);
      const uint32_t both_high = decode_e4m3x2((word_high >> ((chunk & 1) * 16)) & 0x7f7fu);
      const uint32_t multiplier_low[2] = {prmt(both_low, both_low, 0x1010u), prmt(both_low, both_low, 0x3232u)};
      const uint32_t multiplier_high[2] = {prmt(both_high, both_high, 0x1010u),
                                           prmt(both_high, both_high, 0x3232u)};
      const uint32_t words_low[4] = {weights[local][0].x, weights[local][0].y, weights[local][0].z, weights[local][0].w};
      const uint32_t words_high[4] = {weights[local][1].x, weights[local][1].y, weights[local][1].z, weights[local][1].w};
#pragma unroll
      for (int word = 0; word < 4; ++word) {
        uint32_t low[4], high[4];
        decode_e2m1x8_bits(words_low[word], low);
        decode_e2m1x8_bits(words_high[word], high);
        const uint32_t scale_low = multiplier_low[word >> 1];
        const uint32_t scale_high = multiplier_high[word >> 1];
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
          mma_f16_16x8x16(accumulator[step], mul_f16x2(low[2 * pair], scale_low),
                          mul_f16x2(high[2 * pair], scale_high),
                          mul_f16x2(low[2 * pair + 1], scale_low),
                          mul_f16x2(high[2 * pair + 1], scale_high), b[word * 4 + 2 * pair],
                          b[word * 4 + 2 * pair + 1]);
        }
      }
    }
  };

  uint4 weights_even[2][2], weights_odd[2][2];
  uint2 scales_now[2][2], scales_next[2][2];
  uint4 tokens_raw[4];
  if (my_stages > 0) {
    load_weights(first_stage, 0, weights_even);
    load_scales(first_stage, scales_now);
  }
  // Activations may come from the previous kernel of the stream; weights and scales do not.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (my_stages > 0) load_tokens(first_stage, tokens_raw);
  for (int index = 0; index < my_stages; ++index) {
    const int stage = first_stage + index;
    const bool more = index + 1 < my_stages;
    uint32_t b[16];
#pragma unroll
    for (int word = 0; word < 4; ++word) {
      b[word * 4 + 0] = bf16x2_to_f16x2(tokens_raw[word].x);
      b[word * 4 + 1] = bf16x2_to_f16x2(tokens_raw[word].y);
      b[word * 4 + 2] = bf16x2_to_f16x2(tokens_raw[word].z);
      b[word * 4 + 3] = bf16x2_to_f16x2(tokens_raw[word].w);
    }
    load_weights(stage, 1, weights_odd);
    if (more) {
      load_scales(stage + 1, scales_next);
      load_tokens(stage + 1, tokens_raw);
    }
    compute(0, weights_even, scales_now, b);
    if (more) load_weights(stage + 1, 0, weights_even);
    compute(1, weights_odd, scales_now, b);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int row_half = 0; row_half < 2; ++row_half) scales_now[j][row_half] = scales_next[j][row_half];
    }
  }

  // accumulator[step]: rows (group, group + 8) of the step x tokens (2*quad, 2*quad + 1)
#pragma unroll
  for (int step = 0; step < kSteps; ++step) {
    const int row = warp_rows * kRowsPerWarp + step * 16 + group;
    float* base = shared_sums + (warp_k * kTileRows + row) * kMaxTokens + 2 * quad;
    *reinterpret_cast<float2*>(base) = make_float2(accumulator[step][0], accumulator[step][1]);
    *reinterpret_cast<float2*>(base + 8 * kMaxTokens) =
        make_float2(accumulator[step][2], accumulator[step][3]);
  }
  __syncthreads();

  const uint32_t slot_base = ptx::smem_address(shared_parts + part * kTileRows * kMaxTokens);
  const uint32_t remote_base = parts > 1 ? ptx::map_to_cta(slot_base, 0u) : slot_base;
  for (int index = threadIdx.x; index < kTileRows * kMaxTokens; index += kDirectThreads) {
    float sum = shared_sums[index];
#pragma unroll
    for (int sub = 1; sub < kWarpsK; ++sub) sum += shared_sums[sub * kTileRows * kMaxTokens + index];
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_base + index * 4), "f"(sum) : "memory");
  }
  if (parts > 1) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  if (part == 0) {
    for (int index = threadIdx.x; index < kTileRows * kMaxTokens; index += kDirectThreads) {
      const int row = row_tile * kTileRows + index / kMaxTokens;
      const int token = index % kMaxTokens;
      float total = 0.0f;
      for (int slot = 0; slot < parts; ++slot) total += shared_parts[slot * kTileRows * kMaxTokens + index];
      if (row < n && token < m) {
        output[static_cast<size_t>(token) * n + row] = __float2bfloat16_rn(total * global_scale);
      }
    }
  }
}

// K parts (cluster size): the choice that leaves the fewest idle CTA slots. Two CTAs fit on
// an SM; with `parts` parts there are row_tiles * parts CTAs of ceil(stages / parts) stages,
// and the kernel lasts as long as the slot that gets the most of them.
int parts_for(int n, int k, int sm_count) {
  const int row_tiles = (n + kTileRows - 1) / kTileRows;
  const int stages = (k + kStageK - 1) / kStageK;
  const int slots = 2 * sm_count;
  int best = 1;
  long long best_length = 0;
  for (int parts = 1; parts <= kMaxParts && parts <= stages; parts *= 2) {
    const int per_cta = (stages + parts - 1) / parts;
    const long long ctas = static_cast<long long>(row_tiles) * parts;
    const long long rounds = (ctas + slots - 1) / slots;
    const long long length = rounds * per_cta;
    if (parts == 1 || length < best_length) {
      best = parts;
      best_length = length;
    }
  }
  return best;
}

}  // namespace nvfp4_vector
}  // namespace mircuda_b200

extern "C" int mircuda_b200_nvfp4_vector_create(int m, int n, int k, void* stream,
                                                void** output) {
  using namespace mircuda_b200::nvfp4_vector;
  if (m <= 0 || m > kMaxTokens || n <= 0 || k <= 0 || k % 64 != 0 || stream == nullptr ||
      output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->m = m;
  plan->n = n;
  plan->k = k;
  plan->stream = static_cast<cudaStream_t>(stream);
  int sm_count = 0;
  int status = static_cast<int>(cudaGetDevice(&plan->device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, plan->device));
  }
  if (status == 0) {
    status = static_cast<int>(cudaHostAlloc(reinterpret_cast<void**>(&plan->status),
                                            sizeof(uint32_t), cudaHostAllocMapped));
  }
  if (status == 0) {
    status = static_cast<int>(cudaFuncSetAttribute(nvfp4_vector_kernel,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   SharedLayout::kBytes));
  }
  if (status != 0) {
    if (plan->status != nullptr) cudaFreeHost(plan->status);
    delete plan;
    return status;
  }
  *plan->status = 0u;
  plan->parts = parts_for(n, k, sm_count);
  status = static_cast<int>(cudaFuncSetAttribute(nvfp4_direct_kernel<true>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 kDirectSharedBytes));
  if (status == 0) {
    status = static_cast<int>(cudaFuncSetAttribute(nvfp4_direct_kernel<false>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   kDirectSharedBytes));
  }
  if (status != 0) {
    cudaFreeHost(plan->status);
    delete plan;
    return status;
  }
  // Shapes the persistent streaming kernel covers (whole 128-row scale tiles, K a multiple of
  // 2048 up to 12288) run on it; all others on the direct kernel, which measured equal to the
  // ring kernel on large shapes and 6-8 % faster on small ones.
  // MIRCUDA_B200_NVFP4_VECTOR=stream|direct|ring forces a choice (stream only where eligible).
  const char* kernel_choice = std::getenv("MIRCUDA_B200_NVFP4_VECTOR");
  plan->direct = !(kernel_choice != nullptr && std::strcmp(kernel_choice, "ring") == 0);
  const bool forced_other = kernel_choice != nullptr && (std::strcmp(kernel_choice, "ring") == 0 ||
                                                         std::strcmp(kernel_choice, "direct") == 0);
  plan->stream_kernel = !forced_other && mircuda_b200::nvfp4_stream::eligible(n, k);
  if (plan->stream_kernel) {
    status = mircuda_b200::nvfp4_stream::prepare(&plan->stream_config, n, k);
    if (status == -1) {
      plan->stream_kernel = false;      // more tiles per CTA than it keeps running sums for
    } else if (status != 0) {
      cudaFreeHost(plan->status);
      delete plan;
      return status;
    }
  }
  // Overlapped launches (programmatic dependent launch): the kernel may fetch its weights and
  // scales while earlier work of the stream is still running, so that work must not write them
  // (they are model constants); activations are read and outputs written only after it has
  // completed. On by default for the streaming kernel, where it removes about 2 us of launch gap
  // and first-byte latency per call (gate_up 15.6 -> 13.7 us, o 5.8 -> 4.4 us); opt-in for the
  // other two, where it helps single-wave shapes and hurts multi-part ones.
  // MIRCUDA_B200_OVERLAP_LAUNCHES=0 / 1 forces it off / on.
  const char* overlap = std::getenv("MIRCUDA_B200_OVERLAP_LAUNCHES");
  plan->overlap_launches = overlap != nullptr ? overlap[0] == '1' : plan->stream_kernel;
  if (const char* forced = std::getenv("MIRCUDA_B200_NVFP4_PARTS")) {
    const int value = std::atoi(forced);
    const int stages = (k + kStageK - 1) / kStageK;
    if ((value == 1 || value == 2 || value == 4 || value == 8) && value <= stages) plan->parts = value;
  }
  *output = plan;
  return 0;
}

extern "C" int mircuda_b200_nvfp4_vector_execute(void* raw, void* stream, const void* input,
                                                 const void* weight, const void* weight_scales,
                                                 void* output, float global_scale) {
  using namespace mircuda_b200;
  using namespace mircuda_b200::nvfp4_vector;
  if (raw == nullptr || stream == nullptr || input == nullptr || weight == nullptr ||
      weight_scales == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  if (((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(weight_scales) |
        reinterpret_cast<uintptr_t>(input)) & 15u) != 0u) {
    return -1;
  }
  if (plan->stream_kernel) {
    if ((reinterpret_cast<uintptr_t>(output) & 1u) != 0u) return -1;
    return nvfp4_stream::launch(&plan->stream_config, cuda_stream, plan->overlap_launches, input, nullptr,
                                weight, weight_scales, output, plan->m, plan->n, plan->k, global_scale,
                                plan->status);
  }
  if (plan->direct) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((plan->n + kTileRows - 1) / kTileRows, plan->parts, 1);
    config.blockDim = dim3(kDirectThreads, 1, 1);
    config.dynamicSmemBytes = kDirectSharedBytes;
    config.stream = cuda_stream;
    cudaLaunchAttribute attributes[2] = {};
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 1;
    attributes[0].val.clusterDim.y = plan->parts;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = plan->overlap_launches ? 2 : 1;
    auto* kernel = plan->k % kStageK == 0 ? nvfp4_direct_kernel<true> : nvfp4_direct_kernel<false>;
    return static_cast<int>(cudaLaunchKernelEx(
        &config, kernel, static_cast<const uint8_t*>(weight),
        static_cast<const __nv_bfloat16*>(input), static_cast<const uint8_t*>(weight_scales),
        static_cast<__nv_bfloat16*>(output), plan->m, plan->n, plan->k, plan->parts, global_scale));
  }
  if (weight != plan->cached_weight) {
    EncodeTiled encode = encode_tiled_entry();
    if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
    const cuuint64_t dimensions[2] = {static_cast<cuuint64_t>(plan->k / 2), static_cast<cuuint64_t>(plan->n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(plan->k / 2)};
    const cuuint32_t box[2] = {kStageK / 2, kTileRows};
    const cuuint32_t element_strides[2] = {1u, 1u};
    const int status = static_cast<int>(encode(
        &plan->weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2u, const_cast<void*>(weight), dimensions,
        strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    if (status != 0) return status;
    plan->cached_weight = weight;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((plan->n + kTileRows - 1) / kTileRows, plan->parts, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = SharedLayout::kBytes;
  config.stream = cuda_stream;
  cudaLaunchAttribute attributes[2] = {};
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 1;
  attributes[0].val.clusterDim.y = plan->parts;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = plan->overlap_launches ? 2 : 1;
  return static_cast<int>(cudaLaunchKernelEx(
      &config, nvfp4_vector_kernel, plan->weight_map, static_cast<const __nv_bfloat16*>(input),
      static_cast<const uint8_t*>(weight_scales), static_cast<__nv_bfloat16*>(output), plan->m,
      plan->n, plan->k, plan->parts, global_scale, plan->status));
}

extern "C" void mircuda_b200_nvfp4_vector_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::nvfp4_vector::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
