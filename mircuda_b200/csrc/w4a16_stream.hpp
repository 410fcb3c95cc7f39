// Internal interface of the streaming int4-g128 W4A16 decode kernel (w4a16_stream.cu), used by
// the plan entry points in w4a16_int4.cu.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

namespace mircuda_b200 {
namespace w4a16_stream {

struct Config {
  int token_groups;      // groups of 8 tokens (1 or 2)
  int chunks_per_warp;   // 128-element K chunks each consumer warp owns per tile and pass (1 or 2)
  int passes;            // passes over K: k = 2048 * chunks_per_warp * passes
  int ctas;              // persistent CTAs, one per SM (fewer when there are fewer tiles)
};

// m <= 16, n % 16 == 0, k % 2048 == 0; -1 for shapes it does not cover (the caller then uses
// another kernel), another non-zero value for a CUDA error.
int prepare(Config* config, int m, int n, int k);

// `scales` must be 4-byte aligned (a scale travels inside the aligned word that holds it).
int launch(const Config* config, cudaStream_t stream, bool overlap_launches, const void* input,
           const void* weight, const void* scales, void* output, int m, int n, int k, uint32_t* status);

}  // namespace w4a16_stream
}  // namespace mircuda_b200
