// Internal interface of the streaming routed Marlin kernel (marlin_moe_stream.cu), used by
// mircuda_marlin_{nvfp4,mxfp4}_moe_execute in marlin_moe.cu.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

namespace mircuda_b200 {
namespace marlin_moe_stream {

// Shapes the kernel covers: n % 64 == 0, k % 256 == 0 and k <= 2048.
bool eligible(int n, int k);

// Arguments as for the entry points; `block_size` is the route block (8 or 64), `status` a
// host-visible word that is set when a bounded wait ran out (may be null).
int launch(cudaStream_t stream, bool mxfp4, int block_size, const void* input, const void* weight,
           const void* scales, const void* global_scales, void* output, const void* sorted, const void* expert_ids,
           const void* padded, const void* routing, int top_k, bool multiply_routing, int assignments, int n,
           int k, uint32_t* status);

}  // namespace marlin_moe_stream
}  // namespace mircuda_b200
