// Routed W4A16 projections on the Marlin layout: for every assignment id (= token * top_k +
// choice) routed to expert e, output[id, :] = bf16(input[id / top_k, :] . W_e^T * scale_e)
// (optionally times routing[id]), with W_e the expert's NVFP4 or MXFP4 weights repacked into
// Marlin tiles and their prepared scales (marlin_prepare.cu). Routes come from
// mircuda_marlin_prepare_moe_routes: `sorted` lists assignment ids by expert, every expert's
// run padded to the route block size (8 or 64) with the sentinel `assignments`; `expert_ids`
// names the expert of each block; `padded[0]` is the padded length. Replaces the reference's
// vendored Marlin MoE instantiations (sys/native/marlin/moe_kernel.cu:175-205,
// mxfp4_moe_kernel.cu:145-171) behind the same C entry points.
//
// A CTA owns one 64-column tile of N and one group of routed rows that share an expert (the
// 8 rows of a small route block, or 16 of the 64 rows of a large one), walks the whole K in
// rounds of 64 K-tiles with all weight loads of a warp's share in flight together, gathers the
// rows' activations into shared memory per round, and feeds mma.sync.m16n8k16 with the weights
// on the 16-row side (as the dense kernel does). No K slicing, so `temporary`, `locks` and
// `atomic_reduce` are accepted and left untouched; nothing waits on another CTA.
// Numerics: exact weight * scale products in bf16, fp32 accumulation, the expert's prepared
// global scale (NVFP4) applied before the bf16 round. MXFP4 scales are E8M0 bytes; they are
// applied as bf16 powers of two offset by 2^64, which covers scales from 2^-64 to 2^63.
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include <cstdlib>
#include <cstring>

#include "fp4_codec.cuh"
#include "marlin_common.cuh"
#include "marlin_moe_stream.hpp"
#include "marlin_status.hpp"

namespace mircuda_b200 {
namespace marlin_moe {

using namespace marlin;

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kTileN = 64;
constexpr int kTileK = 16;
constexpr int kMaxTilesPerWarp = 8;

// E8M0 byte e -> 2^(e - 127 + 64) as bf16 in both halves (exponent field clamped to 1..254).
__device__ __forceinline__ uint32_t e8m0_multiplier(uint32_t code) {
  const uint32_t field = min(max(code + 64u, 1u), 254u);
  const uint32_t bits = field << 7;
  return bits | (bits << 16);
}

template <int ROW_GROUPS, bool MXFP4>
__global__ void __launch_bounds__(kThreads)
marlin_moe_kernel(const __nv_bfloat16* __restrict__ input, const uint4* __restrict__ weight,
                  const uint8_t* __restrict__ scales, const float* __restrict__ global_scales,
                  __nv_bfloat16* __restrict__ output, const int* __restrict__ sorted,
                  const int* __restrict__ expert_ids, const int* __restrict__ padded,
                  const float* __restrict__ routing, int top_k, bool multiply_routing,
                  int assignments, int n, int k, int block_size) {
  constexpr int kRows = ROW_GROUPS * 8;
  const int first_row = blockIdx.y * kRows;
  if (first_row >= __ldg(padded)) return;
  const int expert = __ldg(expert_ids + first_row / block_size);
  if (expert < 0) return;

  extern __shared__ __align__(16) uint8_t shared_raw[];
  __nv_bfloat16* shared_x = reinterpret_cast<__nv_bfloat16*>(shared_raw);
  const int x_stride = kWarps * kMaxTilesPerWarp * kTileK + 8;
  float* shared_sums = reinterpret_cast<float*>(shared_raw);
  __shared__ int ids[kRows];

  const int tile_n = blockIdx.x;
  const int tiles_n = n / kTileN;
  const int tiles_k = k / kTileK;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int group = lane >> 2;
  const int quad = lane & 3;
  if (threadIdx.x < kRows) ids[threadIdx.x] = __ldg(sorted + first_row + threadIdx.x);

  const size_t expert_words = static_cast<size_t>(tiles_k) * tiles_n * 32;
  const uint4* expert_weight = weight + static_cast<size_t>(expert) * expert_words;
  const int scale_group_tiles = MXFP4 ? 2 : 1;          // K tiles per scale group
  const uint8_t* expert_scales =
      scales + static_cast<size_t>(expert) * n * (tiles_k / scale_group_tiles);

  float accumulator[4][ROW_GROUPS][4];
#pragma unroll
  for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
    for (int rows = 0; rows < ROW_GROUPS; ++rows) {
#pragma unroll
      for (int item = 0; item < 4; ++item) accumulator[quarter][rows][item] = 0.0f;
    }
  }

  constexpr int kRoundTiles = kWarps * kMaxTilesPerWarp;
  for (int round_tile = 0; round_tile < tiles_k; round_tile += kRoundTiles) {
    const int round_tiles = min(kRoundTiles, tiles_k - round_tile);
    uint4 words[kMaxTilesPerWarp];
    uint2 scale_bytes[kMaxTilesPerWarp];
#pragma unroll
    for (int item = 0; item < kMaxTilesPerWarp; ++item) {
      const int local_tile = warp + item * kWarps;
      words[item] = make_uint4(0u, 0u, 0u, 0u);
      scale_bytes[item] = make_uint2(0u, 0u);
      if (local_tile < round_tiles) {
        const int tile_k = round_tile + local_tile;
        words[item] = load_streaming_16(expert_weight + (static_cast<size_t>(tile_k) * tiles_n + tile_n) * 32 + lane);
        scale_bytes[item] = __ldg(reinterpret_cast<const uint2*>(
            expert_scales + static_cast<size_t>(tile_k / scale_group_tiles) * n + tile_n * kTileN + group * 8));
      }
    }

    __syncthreads();   // ids are visible; the previous round's activations are no longer needed
    // Activations of the round in 16-byte pieces (a K tile is two of them).
    const int round_pieces = round_tiles * 2;
    for (int index = threadIdx.x; index < kRows * round_pieces; index += kThreads) {
      const int row = index / round_pieces;
      const int piece = index - row * round_pieces;
      const int id = ids[row];
      uint4 value = make_uint4(0u, 0u, 0u, 0u);
      if (id < assignments) {
        value = __ldg(reinterpret_cast<const uint4*>(
                          input + static_cast<size_t>(id / top_k) * k + round_tile * kTileK) + piece);
      }
      *reinterpret_cast<uint4*>(shared_x + row * x_stride + piece * 8) = value;
    }
    __syncthreads();

#pragma unroll
    for (int item = 0; item < kMaxTilesPerWarp; ++item) {
      const int local_tile = warp + item * kWarps;
      if (local_tile < round_tiles) {
        uint32_t b[ROW_GROUPS][2];
#pragma unroll
        for (int rows = 0; rows < ROW_GROUPS; ++rows) {
          const __nv_bfloat16* x =
              shared_x + (rows * 8 + group) * x_stride + local_tile * kTileK + quad * 2;
          b[rows][0] = *reinterpret_cast<const uint32_t*>(x);
          b[rows][1] = *reinterpret_cast<const uint32_t*>(x + 8);
        }
        const uint32_t quarter_words[4] = {words[item].x, words[item].y, words[item].z, words[item].w};
        // Scale bytes of rows (g, g+8) for quarters 0..3 sit at byte offsets 0,2 | 1,3 | 4,6 | 5,7.
        const uint32_t low = scale_bytes[item].x;
        const uint32_t high = scale_bytes[item].y;
        const uint32_t code[4][2] = {{low & 0xffu, (low >> 16) & 0xffu},
                                     {(low >> 8) & 0xffu, low >> 24},
                                     {high & 0xffu, (high >> 16) & 0xffu},
                                     {(high >> 8) & 0xffu, high >> 24}};
#pragma unroll
        for (int quarter = 0; quarter < 4; ++quarter) {
          uint32_t a[4];
          place_e2m1x8(quarter_words[quarter], a);   // (a0,a1) (a4,a5) (a2,a3) (a6,a7)
          const uint32_t upper = MXFP4 ? e8m0_multiplier(code[quarter][0]) : scale_multiplier(code[quarter][0]);
          const uint32_t lower = MXFP4 ? e8m0_multiplier(code[quarter][1]) : scale_multiplier(code[quarter][1]);
          const uint32_t a0 = mul_bf16x2(a[0], upper);
          const uint32_t a1 = mul_bf16x2(a[2], lower);
          const uint32_t a2 = mul_bf16x2(a[1], upper);
          const uint32_t a3 = mul_bf16x2(a[3], lower);
#pragma unroll
          for (int rows = 0; rows < ROW_GROUPS; ++rows) {
            mma_bf16_16x8x16(accumulator[quarter][rows], a0, a1, a2, a3, b[rows][0], b[rows][1]);
          }
        }
      }
    }
  }
  __syncthreads();   // everyone is done with shared_x; reuse the space for the warp sums

#pragma unroll
  for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
    for (int rows = 0; rows < ROW_GROUPS; ++rows) {
      const int n_local = quarter * 16 + group;
      const int row = rows * 8 + quad * 2;
      float* base = shared_sums + (warp * kTileN + n_local) * kRows + row;
      base[0] = accumulator[quarter][rows][0];
      base[1] = accumulator[quarter][rows][1];
      base[8 * kRows] = accumulator[quarter][rows][2];
      base[8 * kRows + 1] = accumulator[quarter][rows][3];
    }
  }
  __syncthreads();

  // NVFP4: prepared_global * 2^-110 undoes the multiplier's 2^110 and the bit placement's
  // 2^-126 together with the 2^119 / factor folded into the global. MXFP4: 2^(126 - 64).
  const float finish = MXFP4 ? 4.611686018427388e18f
                             : __ldg(global_scales + expert) * 7.70371977754894341e-34f;
  for (int index = threadIdx.x; index < kTileN * kRows; index += kThreads) {
    const int n_local = index % kTileN;
    const int row = index / kTileN;
    const int id = ids[row];
    if (id >= assignments) continue;
    float sum = 0.0f;
#pragma unroll
    for (int part = 0; part < kWarps; ++part) sum += shared_sums[(part * kTileN + n_local) * kRows + row];
    sum *= finish;
    if (multiply_routing) sum *= __ldg(routing + id);
    output[static_cast<size_t>(id) * n + tile_n * kTileN + n_local] = __float2bfloat16_rn(sum);
  }
}

template <bool MXFP4>
int execute(void* stream, const void* input, const void* weight, void* output, const void* scales,
            const void* global_scales, const void* sorted, const void* expert_ids,
            const void* padded, const void* routing, int top_k, bool multiply_routing, int tokens,
            int n, int k, int thread_config) {
  if (stream == nullptr || input == nullptr || weight == nullptr || output == nullptr ||
      scales == nullptr || sorted == nullptr || expert_ids == nullptr || padded == nullptr ||
      routing == nullptr || (!MXFP4 && global_scales == nullptr) || top_k <= 0 || tokens <= 0 ||
      n <= 0 || k <= 0 || n % kTileN != 0 || k % (MXFP4 ? 32 : kTileK) != 0 || thread_config < 0 ||
      thread_config > 5 || (reinterpret_cast<uintptr_t>(input) & 15u) != 0u) {
    return -1;
  }
  // Thread configurations 0-2 route in blocks of 8 rows, 3-5 in blocks of 64
  // (src/marlin/spec.rs:100-105).
  const int block_size = thread_config < 3 ? 8 : 64;
  const long long assignments = static_cast<long long>(tokens) * top_k;
  // Shapes the streaming kernel covers go to it, except short K with few routed rows, where its
  // per-unit costs outweigh what it streams (K = 768 x N = 2048, one token: 7.3 against 6.2 us).
  // MIRCUDA_B200_MARLIN_MOE=tiles / stream forces the tile kernel below / the streaming kernel.
  const char* choice = std::getenv("MIRCUDA_B200_MARLIN_MOE");
  const bool forced_stream = choice != nullptr && std::strcmp(choice, "stream") == 0;
  if ((choice == nullptr || forced_stream) && (forced_stream || k >= 1024 || assignments >= 32) &&
      marlin_moe_stream::eligible(n, k) &&
      assignments < (1ll << 31) && (reinterpret_cast<uintptr_t>(weight) & 15u) == 0u &&
      (reinterpret_cast<uintptr_t>(scales) & 7u) == 0u) {
    bool failed = false;
    uint32_t* status_word = marlin_status_word(static_cast<cudaStream_t>(stream), &failed);
    if (failed) return -3;
    return marlin_moe_stream::launch(static_cast<cudaStream_t>(stream), MXFP4, block_size, input, weight, scales,
                                     global_scales, output, sorted, expert_ids, padded, routing, top_k,
                                     multiply_routing, static_cast<int>(assignments), n, k, status_word);
  }
  // The padded length is only known on the device; the grid covers its upper bound
  // (assignments + one partly filled block per expert is at most assignments * block_size).
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  const int x_stride = kWarps * kMaxTilesPerWarp * kTileK + 8;
  if (block_size == 8) {
    const long long groups = assignments;                       // every block holds >= 1 id
    const size_t shared = sizeof(__nv_bfloat16) * 8 * x_stride > sizeof(float) * kWarps * kTileN * 8
                              ? sizeof(__nv_bfloat16) * 8 * x_stride
                              : sizeof(float) * kWarps * kTileN * 8;
    marlin_moe_kernel<1, MXFP4><<<dim3(n / kTileN, static_cast<unsigned int>(groups), 1), kThreads, shared, cuda_stream>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<const uint4*>(weight),
        static_cast<const uint8_t*>(scales), static_cast<const float*>(global_scales),
        static_cast<__nv_bfloat16*>(output), static_cast<const int*>(sorted),
        static_cast<const int*>(expert_ids), static_cast<const int*>(padded),
        static_cast<const float*>(routing), top_k, multiply_routing, static_cast<int>(assignments), n,
        k, block_size);
  } else {
    const long long groups = assignments * 4;                   // 64-row blocks, 16 rows a CTA
    const size_t shared = sizeof(__nv_bfloat16) * 16 * x_stride > sizeof(float) * kWarps * kTileN * 16
                              ? sizeof(__nv_bfloat16) * 16 * x_stride
                              : sizeof(float) * kWarps * kTileN * 16;
    marlin_moe_kernel<2, MXFP4><<<dim3(n / kTileN, static_cast<unsigned int>(groups), 1), kThreads, shared, cuda_stream>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<const uint4*>(weight),
        static_cast<const uint8_t*>(scales), static_cast<const float*>(global_scales),
        static_cast<__nv_bfloat16*>(output), static_cast<const int*>(sorted),
        static_cast<const int*>(expert_ids), static_cast<const int*>(padded),
        static_cast<const float*>(routing), top_k, multiply_routing, static_cast<int>(assignments), n,
        k, block_size);
  }
  return static_cast<int>(cudaPeekAtLastError());
}

}  // namespace marlin_moe
}  // namespace mircuda_b200

extern "C" int mircuda_marlin_nvfp4_moe_execute(
    void* stream, const void* input, const void* weight, void* output, void* temporary,
    const void* scales, const void* global_scales, const void* sorted, const void* expert_ids,
    const void* padded, const void* routing, int top_k, bool multiply_routing, int tokens,
    int output_features, int input_features, int thread_config, void* locks, bool atomic_reduce) {
  (void)temporary;
  (void)locks;
  (void)atomic_reduce;
  return mircuda_b200::marlin_moe::execute<false>(stream, input, weight, output, scales,
                                                  global_scales, sorted, expert_ids, padded, routing,
                                                  top_k, multiply_routing, tokens, output_features,
                                                  input_features, thread_config);
}

extern "C" int mircuda_marlin_mxfp4_moe_execute(
    void* stream, const void* input, const void* weight, void* output, void* temporary,
    const void* scales, const void* sorted, const void* expert_ids, const void* padded,
    const void* routing, int top_k, bool multiply_routing, int tokens, int output_features,
    int input_features, int thread_config, void* locks, bool atomic_reduce) {
  (void)temporary;
  (void)locks;
  (void)atomic_reduce;
  return mircuda_b200::marlin_moe::execute<true>(stream, input, weight, output, scales, nullptr,
                                                 sorted, expert_ids, padded, routing, top_k,
                                                 multiply_routing, tokens, output_features,
                                                 input_features, thread_config);
}
