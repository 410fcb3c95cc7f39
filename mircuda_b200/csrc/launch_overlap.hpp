// Whether kernels that begin with a dependency wait are launched with programmatic stream
// serialisation, so that their set-up overlaps the tail of the kernel before them on the stream.
// Those kernels touch no global memory before the wait, so the caller sees plain stream order
// either way. MIRCUDA_B200_OVERLAP_LAUNCHES=0 turns it off.
#pragma once

#include <cstdlib>

namespace mircuda_b200 {

inline bool overlap_launches() {
  static const bool enabled = [] {
    const char* value = std::getenv("MIRCUDA_B200_OVERLAP_LAUNCHES");
    return value == nullptr || value[0] != '0';
  }();
  return enabled;
}

}  // namespace mircuda_b200
