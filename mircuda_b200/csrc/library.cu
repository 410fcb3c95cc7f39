// Library identification.
#include <cstdint>

extern "C" uint32_t mircuda_b200_version(void) { return (0u << 16) | (1u << 8) | 0u; }
