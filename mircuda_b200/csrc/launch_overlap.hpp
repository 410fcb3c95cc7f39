// Whether kernels that begin with a dependency wait are launched with programmatic stream
// serialisation, so that their set-up overlaps the tail of the kernel before them on the stream.
// Those kernels touch no global memory before the wait, so the caller sees plain stream order
// either way. MIRCUDA_B200_OVERLAP_LAUNCHES=0 turns it off.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>

namespace mircuda_b200 {

inline bool overlap_launches() {
  static const bool enabled = [] {
    const char* value = std::getenv("MIRCUDA_B200_OVERLAP_LAUNCHES");
    return value == nullptr || value[0] != '0';
  }();
  return enabled;
}

#ifdef __CUDACC__
// Launches `kernel` so that it may be scheduled while the kernel before it on the stream is still
// finishing (when overlap_launches() says so). Only for kernels that execute a dependency wait
// before their first access to global memory.
template <typename... Parameters, typename... Arguments>
inline int launch_after_dependency(void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes,
                                   cudaStream_t stream, Arguments... arguments) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = overlap_launches() ? 1u : 0u;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, static_cast<Parameters>(arguments)...));
}
#endif

}  // namespace mircuda_b200
