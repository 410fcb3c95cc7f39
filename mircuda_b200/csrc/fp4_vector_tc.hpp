// Tensor-core implementation of the FP4 x FP4 GEMV behind mircuda_fp4_vector_* (fp4_vector.cu
// owns the C entry points and picks between this and its CUDA-core kernel).
#pragma once

#include <cuda_runtime_api.h>

namespace mircuda_b200 {
namespace fp4_vector_tc {

struct Plan;

// n > 0, k a positive multiple of 64. Allocations are made on `stream`.
int create(int n, int k, cudaStream_t stream, Plan** output);
// input, weight and both scale pointers 16-byte aligned. Returns -3 after a launch whose
// bounded wait ran out.
int execute(Plan* plan, cudaStream_t stream, const void* input, const void* input_scales,
            const void* weight, const void* weight_scales, void* output, float alpha);
void destroy(Plan* plan);

}  // namespace fp4_vector_tc
}  // namespace mircuda_b200
