// Internal interface of the fused int4 W4A16 prefill GEMM (w4a16_tile.cu), used by the plan entry
// points in w4a16_int4.cu.
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>

namespace mircuda_b200 {
namespace w4a16_tile {

struct Config {
  bool pair;                   // CTA pairs (w4a16_pair.cu, 256-token tiles) or single CTAs (128-token tiles)
  int resident_pairs;          // pairs the device can hold at once
  int sm_count;
  int splits;                  // K ranges per tile; more than one needs the workspace
  size_t workspace_bytes;      // splits * m * n floats when splits > 1, else 0
  const void* cached_input;    // operands the tensor maps below were encoded for
  const void* cached_weight;
  CUtensorMap map_a, map_w;
};

// Shapes the kernel covers: n % 8 == 0 (16-byte output rows) and whole scale groups along K.
bool eligible(int m, int n, int k);

// Sets the kernel attribute, reads the device's SM count and decides the K split.
int prepare(Config* config, int m, int n, int k);

// input f16 [m, k], weight bytes [n, k / 2], scales f16 [n, k / 128], output f16 [m, n]; all
// 16-byte aligned except the scales (2 bytes). `workspace`: workspace_bytes of device memory.
int launch(Config* config, cudaStream_t stream, const void* input, const void* weight, const void* scales,
           void* output, void* workspace, int m, int n, int k, uint32_t* status_word);

// The CTA-pair kernel (w4a16_pair.cu): attribute and occupancy at plan creation, launch with the
// tensor maps of `config` already encoded.
int prepare_pair(Config* config);
int launch_pair(Config* config, cudaStream_t stream, const void* scales, void* output, void* workspace, int m,
                int n, int k, uint32_t* status_word);

}  // namespace w4a16_tile
}  // namespace mircuda_b200
