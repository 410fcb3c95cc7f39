// TEST INFRASTRUCTURE ONLY — never part of the product library.
//
// Builds the reference's own run-time-compiled kernels (kernels/mxfp8.cu) ahead of time
// for sm_100a, from where the file lies in the reference checkout
// (-DREF_MXFP8_CU=...), and adds launchers that use exactly the launch geometry the
// reference's Rust host code chooses. The result is the on-GPU reference the CUDA path is
// compared with bit for bit. These kernels are plain SIMT code without waits or locks.
#include <cuda_runtime_api.h>

#ifndef REF_MXFP8_CU
#error "pass -DREF_MXFP8_CU=\"<reference>/kernels/mxfp8.cu\""
#endif

#include REF_MXFP8_CU

extern "C" {

// Geometry from src/mxfp8/tensor_core.rs:142-151: grid (K/32, M), one warp per block.
int ref_mxfp8_quantize_bf16(const void* input, void* output, void* scales, unsigned int rows,
                            unsigned int columns, void* stream) {
  dim3 grid(columns / 32u, rows, 1u);
  mircuda_mxfp8_quantize_bf16<<<grid, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned short*>(input), static_cast<unsigned char*>(output),
      static_cast<unsigned char*>(scales), rows, columns);
  return static_cast<int>(cudaPeekAtLastError());
}

// Geometry from src/mxfp8/tensor_core.rs:101-105: one thread per element, 256 per block.
int ref_mxfp8_swizzle_scales(const void* input, void* output, unsigned int rows,
                             unsigned int columns, void* stream) {
  unsigned int elements = rows * columns;
  mircuda_mxfp8_swizzle_scales<<<(elements + 255u) / 256u, 256, 0,
                                 static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(input), static_cast<unsigned char*>(output), rows, columns);
  return static_cast<int>(cudaPeekAtLastError());
}

// Geometry from src/mxfp8/matmul.rs:131-157: grid (N, tokens) or (N, ceil(tokens/4)), 256 threads.
int ref_mxfp8_bf16(const void* input, const void* weight, const void* scales, void* output,
                   unsigned int tokens, unsigned int input_features, unsigned int output_features,
                   int tiled, void* stream) {
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (tiled) {
    dim3 grid(output_features, (tokens + 3u) / 4u, 1u);
    mircuda_mxfp8_bf16_tiled<<<grid, 256, 0, cuda_stream>>>(
        static_cast<const unsigned short*>(input), static_cast<const unsigned int*>(weight),
        static_cast<const unsigned char*>(scales), static_cast<unsigned short*>(output), tokens,
        input_features, output_features);
  } else {
    dim3 grid(output_features, tokens, 1u);
    mircuda_mxfp8_bf16<<<grid, 256, 0, cuda_stream>>>(
        static_cast<const unsigned short*>(input), static_cast<const unsigned int*>(weight),
        static_cast<const unsigned char*>(scales), static_cast<unsigned short*>(output), tokens,
        input_features, output_features);
  }
  return static_cast<int>(cudaPeekAtLastError());
}

}  // extern "C"
