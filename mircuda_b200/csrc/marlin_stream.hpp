// Internal interface of the streaming Marlin-layout NVFP4 decode kernel (marlin_stream.cu), used
// by mircuda_marlin_nvfp4_dense_execute in marlin_dense.cu.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

namespace mircuda_b200 {
namespace marlin_stream {

struct Config {
  int row_groups;        // 1: tokens <= 8, 2: tokens <= 16
  int chunks_per_warp;   // 512-element K parts a consumer warp holds activation fragments for
  int slices;            // K slices of one N tile, met through the caller's `temporary` / `locks`
  int passes;            // passes over K inside a CTA: k = 512 * chunks_per_warp * passes * slices
  int ctas;              // persistent CTAs, one per SM (fewer when there are fewer units)
};

// Picks the split of K and sets the kernel attributes; -1 when the shape is not covered (N not a
// multiple of 64, K not a multiple of 512, operands of 4 GB or more, or more running sums than the kernel keeps): the
// caller then uses the tile kernel.
int prepare(Config* config, int tokens, int n, int k, int sm_count);

int launch(const Config& config, cudaStream_t stream, bool overlap_launches, const void* input,
           const void* weight, const void* scales, const float* global_scale, void* output,
           void* temporary, void* locks, int tokens, int n, int k, uint32_t* status);

}  // namespace marlin_stream
}  // namespace mircuda_b200
