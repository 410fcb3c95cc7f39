// TEST INFRASTRUCTURE ONLY — never part of the product library.
//
// Compiles the reference's own kernels/mxfp8.cu for the HOST, from where it lies in the
// reference checkout (path given by -DREF_MXFP8_CU=...), so that its plain-C helper
// functions (bf16 conversion, E4M3/E8M0 codec, scale offset) can be called directly to
// pin the C restatement in mircuda_oracle.c. The __global__ kernels in that file are
// compiled as ordinary functions against inert stand-ins for the CUDA built-ins and are
// never called: a single host thread cannot reproduce their warp shuffles.
#include <algorithm>
#include <cmath>
#include <cstring>

#ifndef REF_MXFP8_CU
#error "pass -DREF_MXFP8_CU=\"<reference>/kernels/mxfp8.cu\""
#endif

#define __device__
#define __global__
#define __shared__ static

namespace {
struct Index3 {
  unsigned int x, y, z;
};
thread_local Index3 blockIdx{0, 0, 0}, threadIdx{0, 0, 0}, blockDim{1, 1, 1};

inline float __uint_as_float(unsigned int bits) {
  float value;
  std::memcpy(&value, &bits, sizeof value);
  return value;
}
inline float __int_as_float(int bits) {
  float value;
  std::memcpy(&value, &bits, sizeof value);
  return value;
}
inline unsigned int __float_as_uint(float value) {
  unsigned int bits;
  std::memcpy(&bits, &value, sizeof bits);
  return bits;
}
inline float __shfl_down_sync(unsigned int, float value, unsigned int) { return value; }
inline float __shfl_sync(unsigned int, float value, unsigned int) { return value; }
inline void __syncthreads() {}
using std::max;
using std::min;
}  // namespace

#include REF_MXFP8_CU

extern "C" {
float ref_bf16_to_float(unsigned short value) { return mircuda_bf16_to_float(value); }
unsigned short ref_float_to_bf16(float value) { return mircuda_float_to_bf16(value); }
float ref_e4m3(unsigned char value) { return mircuda_e4m3(value); }
float ref_e8m0(unsigned char value) { return mircuda_e8m0(value); }
unsigned char ref_encode_e4m3(float value) { return mircuda_encode_e4m3(value); }
unsigned int ref_scale_offset(unsigned int row, unsigned int column, unsigned int rows,
                              unsigned int columns) {
  return mircuda_mxfp8_scale_offset(row, column, rows, columns);
}
}
