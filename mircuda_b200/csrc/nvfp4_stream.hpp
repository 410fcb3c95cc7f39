// Internal interface of the streaming bf16 x NVFP4 decode kernel (nvfp4_stream.cu), used by
// the plan entry points in nvfp4_vector.cu.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

namespace mircuda_b200 {
namespace nvfp4_stream {

struct Config {
  int chunks_per_warp;   // 128-element K chunks each consumer warp owns per tile and pass (1..3)
  int passes;            // passes over K: k = 2048 * chunks_per_warp * passes
  int ctas;              // persistent CTAs, one per SM (fewer when there are fewer tiles)
};

// Shapes the kernel covers: whole 128-row scale tiles and K a multiple of 2048.
bool eligible(int n, int k);

// Picks the split of K into passes and chunks per warp and sets the kernel attributes; -1 when
// the shape needs more running sums than the kernel keeps (the caller then uses another kernel).
int prepare(Config* config, int n, int k);

// `input_scales` null: `input` is bf16 [m, k]. Otherwise `input` is one NVFP4 vector (k / 2 code
// bytes) with its swizzled block scales, and m must be 1.
int launch(Config* config, cudaStream_t stream, bool overlap_launches, const void* input,
           const void* input_scales, const void* weight, const void* weight_scales, void* output, int m,
           int n, int k, float global_scale, uint32_t* status);

}  // namespace nvfp4_stream
}  // namespace mircuda_b200
