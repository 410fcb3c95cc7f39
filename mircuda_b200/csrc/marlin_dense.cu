// W4A16 dense projection on the Marlin layout for decode: bf16 activations [tokens <= 16, K]
// times NVFP4 weights that were repacked into Marlin tiles (marlin_prepare.cu) with their
// group-16 scales prepared into the permuted 8-bit form, to bf16 [tokens, N]. Replaces the
// reference's vendored Marlin kernel instantiation (sys/native/marlin/dense_kernel.cu:73-102)
// behind the same C entry point. Numerics: exact weight * scale products in bf16, fp32
// accumulation, the prepared global scale applied before the bf16 round (the reference's
// epilogue, sys/native/marlin/vendor/dense_template.h:1655-1658).
//
// The op streams N*K/2 + N*K/16 bytes once and is bound by HBM. One packed u32 is already
// one thread's A fragment of mma.sync.m16n8k16 for a 16-row x 16-column weight block, so a
// lane's 16-byte load covers four such blocks (64 output rows) of one 16-wide K tile, and its
// eight scale bytes are 8 adjacent bytes. A CTA owns one 64-row tile of N and a K slice; its
// eight warps take the slice's K tiles round-robin, each with a rolling window of four tiles'
// loads in flight (weights, scales and its activation fragments straight from L1/L2; no barrier
// in the loop), then add their accumulators through shared memory. K slices of one N tile meet in
// the caller's `temporary` buffer; the slice that arrives last (a counter in the caller's
// `locks`, which stay zero between launches) adds them in a fixed order. Nothing spins.
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include <cstdlib>
#include <cstring>

#include "fp4_codec.cuh"
#include "launch_overlap.hpp"
#include "marlin_common.cuh"
#include "marlin_status.hpp"
#include "marlin_stream.hpp"
#include "ptx.cuh"

namespace mircuda_b200 {
namespace marlin_dense {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kTileN = 64;
constexpr int kTileK = 16;
constexpr int kMaxTokens = 16;
constexpr int kAhead = 4;                  // K tiles whose loads one warp keeps in flight

using namespace marlin;

template <int ROW_GROUPS>   // 1: tokens <= 8, 2: tokens <= 16
__global__ void __launch_bounds__(kThreads)
marlin_nvfp4_dense_kernel(const __nv_bfloat16* __restrict__ input,
                          const uint4* __restrict__ weight, const uint8_t* __restrict__ scales,
                          const float* __restrict__ global_scale,
                          __nv_bfloat16* __restrict__ output, float* __restrict__ temporary,
                          int* __restrict__ locks, int tokens, int n, int k, int slices,
                          int tiles_per_slice) {
  extern __shared__ __align__(16) uint8_t shared_raw[];
  constexpr int kRows = ROW_GROUPS * 8;
  float* shared_sums = reinterpret_cast<float*>(shared_raw);   // the warps' sums meet here
  __shared__ bool last_arrival;

  const int tile_n = blockIdx.x;
  const int slice = blockIdx.y;
  const int tiles_n = n / kTileN;
  const int first_tile_k = slice * tiles_per_slice;
  const int tiles_k_total = k / kTileK;
  const int tiles_here = min(tiles_per_slice, tiles_k_total - first_tile_k);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int group = lane >> 2;
  const int quad = lane & 3;

  float accumulator[4][ROW_GROUPS][4];
#pragma unroll
  for (int quarter = 0; quarter < 4; ++quarter) {
#pragma unroll
    for (int rows = 0; rows < ROW_GROUPS; ++rows) {
#pragma unroll
      for (int item = 0; item < 4; ++item) accumulator[quarter][rows][item] = 0.0f;
    }
  }

  // This warp's K tiles of the slice: warp, warp + 8, ... Nothing in the loop is shared between
  // warps (activations come straight from L1/L2: the slice of x is at most 64 KB and every warp
  // and CTA of the SM reads it), so there is no barrier and each warp keeps a rolling window of
  // kAhead tiles' loads in flight: the loads for tile i + kAhead go out before tile i is used.
  const int my_tiles = tiles_here > warp ? (tiles_here - warp + kWarps - 1) / kWarps : 0;
  const uint4* weight_lane = weight + (static_cast<size_t>(first_tile_k + warp) * tiles_n + tile_n) * 32 + lane;
  const uint8_t* scale_lane = scales + static_cast<size_t>(first_tile_k + warp) * n + tile_n * kTileN + group * 8;
  const size_t weight_step = static_cast<size_t>(kWarps) * tiles_n * 32;      // uint4 per K-tile step
  const size_t scale_step = static_cast<size_t>(kWarps) * n;
  const __nv_bfloat16* x_lane = input + static_cast<size_t>(group) * k + (first_tile_k + warp) * kTileK + quad * 2;
  bool row_valid[ROW_GROUPS];
#pragma unroll
  for (int rows = 0; rows < ROW_GROUPS; ++rows) row_valid[rows] = rows * 8 + group < tokens;

  uint4 words[kAhead];
  uint2 scale_bytes[kAhead];
  uint32_t x_low[kAhead][ROW_GROUPS], x_high[kAhead][ROW_GROUPS];
  auto fetch = [&](int slot, int item) {
    words[slot] = make_uint4(0u, 0u, 0u, 0u);
    scale_bytes[slot] = make_uint2(0u, 0u);
#pragma unroll
    for (int rows = 0; rows < ROW_GROUPS; ++rows) x_low[slot][rows] = x_high[slot][rows] = 0u;
    if (item < my_tiles) {
      words[slot] = load_streaming_16(weight_lane + item * weight_step);
      scale_bytes[slot] = __ldg(reinterpret_cast<const uint2*>(scale_lane + item * scale_step));
#pragma unroll
      for (int rows = 0; rows < ROW_GROUPS; ++rows) {
        if (row_valid[rows]) {
          const __nv_bfloat16* x = x_lane + static_cast<size_t>(rows) * 8 * k + item * (kWarps * kTileK);
          x_low[slot][rows] = __ldg(reinterpret_cast<const uint32_t*>(x));
          x_high[slot][rows] = __ldg(reinterpret_cast<const uint32_t*>(x + 8));
        }
      }
    }
  };
#pragma unroll
  for (int slot = 0; slot < kAhead; ++slot) fetch(slot, slot);

  for (int base = 0; base < my_tiles; base += kAhead) {
#pragma unroll
    for (int slot = 0; slot < kAhead; ++slot) {
      const uint4 word = words[slot];
      const uint2 scale = scale_bytes[slot];
      uint32_t b[ROW_GROUPS][2];
#pragma unroll
      for (int rows = 0; rows < ROW_GROUPS; ++rows) {
        b[rows][0] = x_low[slot][rows];
        b[rows][1] = x_high[slot][rows];
      }
      fetch(slot, base + slot + kAhead);
      // A tile past the end carries zero words and zero scale codes: it adds nothing.
      const uint32_t quarter_words[4] = {word.x, word.y, word.z, word.w};
      // Scale bytes of rows (g, g+8) for quarters 0..3 sit at byte offsets 0,2 | 1,3 | 4,6 | 5,7.
      const uint32_t low = scale.x;
      const uint32_t high = scale.y;
      const uint32_t code[4][2] = {{low & 0xffu, (low >> 16) & 0xffu},
                                   {(low >> 8) & 0xffu, low >> 24},
                                   {high & 0xffu, (high >> 16) & 0xffu},
                                   {(high >> 8) & 0xffu, high >> 24}};
#pragma unroll
      for (int quarter = 0; quarter < 4; ++quarter) {
        uint32_t a[4];
        place_e2m1x8(quarter_words[quarter], a);   // (a0,a1) (a4,a5) (a2,a3) (a6,a7)
        const uint32_t upper = scale_multiplier(code[quarter][0]);   // row g
        const uint32_t lower = scale_multiplier(code[quarter][1]);   // row g + 8
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

  // shared_sums[warp][n_local 0..63][row 0..kRows-1]
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

  // finish = prepared_global * 2^-110 undoes the 2^110 of the multiplier and the 2^-126 of
  // the bit placement (2^-16 in total) together with the 2^119 / factor folded into the global.
  const float finish = *global_scale * 7.70371977754894341e-34f;   // 2^-110
  for (int index = threadIdx.x; index < kTileN * kRows; index += kThreads) {
    const int n_local = index / kRows;
    const int row = index % kRows;
    float sum = 0.0f;
#pragma unroll
    for (int part = 0; part < kWarps; ++part) sum += shared_sums[(part * kTileN + n_local) * kRows + row];
    const int column = tile_n * kTileN + n_local;
    if (slices == 1) {
      if (row < tokens) output[static_cast<size_t>(row) * n + column] = __float2bfloat16_rn(sum * finish);
    } else {
      temporary[(static_cast<size_t>(slice) * n + column) * kMaxTokens + row] = sum;
    }
  }
  if (slices == 1) return;

  ptx::fence_acq_rel_gpu();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(&locks[tile_n], 1);
    last_arrival = arrived == slices - 1;
    if (last_arrival) locks[tile_n] = 0;
  }
  __syncthreads();
  if (!last_arrival) return;
  ptx::fence_acq_rel_gpu();
  for (int index = threadIdx.x; index < kTileN * kRows; index += kThreads) {
    const int n_local = index / kRows;
    const int row = index % kRows;
    const int column = tile_n * kTileN + n_local;
    float total = 0.0f;
    for (int part = 0; part < slices; ++part) {
      total += __ldcg(temporary + (static_cast<size_t>(part) * n + column) * kMaxTokens + row);
    }
    if (row < tokens) output[static_cast<size_t>(row) * n + column] = __float2bfloat16_rn(total * finish);
  }
}

}  // namespace marlin_dense
}  // namespace mircuda_b200

extern "C" int mircuda_marlin_nvfp4_dense_execute(void* stream, const void* input,
                                                  const void* weight, void* output,
                                                  void* temporary, const void* scales,
                                                  const float* global_scale, int tokens,
                                                  int output_features, int input_features,
                                                  int thread_config, void* locks,
                                                  bool atomic_reduce) {
  using namespace mircuda_b200::marlin_dense;
  (void)thread_config;   // the tile geometry of this kernel is fixed
  (void)atomic_reduce;   // the cross-slice reduction is always the ordered one
  if (stream == nullptr || input == nullptr || weight == nullptr || output == nullptr ||
      temporary == nullptr || scales == nullptr || global_scale == nullptr || locks == nullptr ||
      tokens <= 0 || tokens > kMaxTokens || output_features <= 0 || input_features <= 0 ||
      output_features % kTileN != 0 || input_features % kTileK != 0 ||
      (reinterpret_cast<uintptr_t>(input) & 15u) != 0u) {
    return -1;
  }
  int device = 0, sm_count = 0;
  int status = static_cast<int>(cudaGetDevice(&device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  }
  if (status != 0) return status;
  // Shapes the streaming kernel covers go to it (MIRCUDA_B200_MARLIN_DENSE=tiles keeps the tile
  // kernel below). Its bounded waits report through the process-wide status word.
  const char* choice = std::getenv("MIRCUDA_B200_MARLIN_DENSE");
  if (choice == nullptr || std::strcmp(choice, "tiles") != 0) {
    bool failed = false;
    uint32_t* stream_status = mircuda_b200::marlin_status_word(static_cast<cudaStream_t>(stream), &failed);
    if (failed) return -3;
    mircuda_b200::marlin_stream::Config config = {};
    if ((reinterpret_cast<uintptr_t>(weight) & 15u) == 0u && (reinterpret_cast<uintptr_t>(scales) & 7u) == 0u &&
        (reinterpret_cast<uintptr_t>(temporary) & 15u) == 0u &&
        mircuda_b200::marlin_stream::prepare(&config, tokens, output_features, input_features, sm_count) == 0) {
      return mircuda_b200::marlin_stream::launch(
          config, static_cast<cudaStream_t>(stream), mircuda_b200::overlap_launches(), input, weight, scales,
          global_scale, output, temporary, locks, tokens, output_features, input_features, stream_status);
    }
  }
  const int tiles_n = output_features / kTileN;
  const int tiles_k = input_features / kTileK;
  // K slices: enough CTAs to fill the machine twice over, each with at least 8 K tiles.
  // Slices need one lock per N tile (the caller provides one per SM) and
  // slices * N * 16 floats of `temporary` (the caller provides 4096 per SM); a shape that
  // does not fit runs unsliced.
  int slices = (2 * sm_count + tiles_n - 1) / tiles_n;
  if (slices > tiles_k / kWarps) slices = tiles_k / kWarps > 0 ? tiles_k / kWarps : 1;
  const long long capacity = static_cast<long long>(sm_count) * 4096;
  if (tiles_n > sm_count) slices = 1;
  while (slices > 1 && static_cast<long long>(slices) * output_features * kMaxTokens > capacity) {
    --slices;
  }
  int tiles_per_slice = (tiles_k + slices - 1) / slices;
  slices = (tiles_k + tiles_per_slice - 1) / tiles_per_slice;
  const dim3 grid(tiles_n, slices);
  const int rows = tokens <= 8 ? 8 : 16;
  const size_t shared_bytes = static_cast<size_t>(kWarps) * kTileN * rows * sizeof(float);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (tokens <= 8) {
    marlin_nvfp4_dense_kernel<1><<<grid, kThreads, shared_bytes, cuda_stream>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<const uint4*>(weight),
        static_cast<const uint8_t*>(scales), global_scale, static_cast<__nv_bfloat16*>(output),
        static_cast<float*>(temporary), static_cast<int*>(locks), tokens, output_features,
        input_features, slices, tiles_per_slice);
  } else {
    marlin_nvfp4_dense_kernel<2><<<grid, kThreads, shared_bytes, cuda_stream>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<const uint4*>(weight),
        static_cast<const uint8_t*>(scales), global_scale, static_cast<__nv_bfloat16*>(output),
        static_cast<float*>(temporary), static_cast<int*>(locks), tokens, output_features,
        input_features, slices, tiles_per_slice);
  }
  return static_cast<int>(cudaPeekAtLastError());
}
