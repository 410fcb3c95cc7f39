// Dense GEMV for decode: y[N] = alpha * W[N,K] x[K] + beta * y, bf16 or f16 storage, fp32
// accumulation. Replaces sys/native/dense_vector_sm120.cu behind the same C entry points.
//
// The op streams W once (2*N*K bytes) and is bound by HBM. One warp owns two rows at a time;
// every lane issues 16-byte streaming loads, four per row in flight, and the activation
// vector comes through L1 (it is a few KB and shared by every warp of the SM). Rows are
// reduced with warp shuffles. Grids are sized so that all warps are resident at once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <new>

namespace mircuda_b200 {
namespace dense_vector {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 2;
constexpr int kUnroll = 4;

struct Plan {
  int data_type;
  int n;
  int k;
  cudaStream_t stream;
};

template <typename T>
struct Convert;

template <>
struct Convert<__half> {
  __device__ static float2 pair(uint32_t bits) {
    return __half22float2(*reinterpret_cast<const __half2*>(&bits));
  }
  __device__ static float one(__half value) { return __half2float(value); }
  __device__ static __half from(float value) { return __float2half_rn(value); }
};

template <>
struct Convert<__nv_bfloat16> {
  __device__ static float2 pair(uint32_t bits) {
    return make_float2(__uint_as_float(bits << 16), __uint_as_float(bits & 0xffff0000u));
  }
  __device__ static float one(__nv_bfloat16 value) { return __bfloat162float(value); }
  __device__ static __nv_bfloat16 from(float value) { return __float2bfloat16_rn(value); }
};

__device__ __forceinline__ uint4 load_streaming(const uint4* pointer) {
  uint4 value;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
               : "l"(pointer));
  return value;
}

template <typename T>
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float sum) {
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
  const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    const float2 a = Convert<T>::pair(xs[pair]);
    const float2 b = Convert<T>::pair(ws[pair]);
    sum = fmaf(a.x, b.x, sum);
    sum = fmaf(a.y, b.y, sum);
  }
  return sum;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
dense_vector_kernel(const T* __restrict__ input, const T* __restrict__ weight, T* __restrict__ output, int n,
       int k, float alpha, float beta) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int first_row = (blockIdx.x * kWarps + warp) * kRowsPerWarp;
  if (first_row >= n) return;
  float sums[kRowsPerWarp] = {};

  if ((k & 7) == 0 && (reinterpret_cast<uintptr_t>(weight) & 15u) == 0 &&
      (reinterpret_cast<uintptr_t>(input) & 15u) == 0) {
    const int vectors = k / 8;
    const uint4* x = reinterpret_cast<const uint4*>(input);
    const uint4* rows[kRowsPerWarp];
#pragma unroll
    for (int item = 0; item < kRowsPerWarp; ++item) {
      const int row = min(first_row + item, n - 1);
      rows[item] = reinterpret_cast<const uint4*>(weight + static_cast<size_t>(row) * k);
    }
    int vector = lane;
    for (; vector + 32 * (kUnroll - 1) < vectors; vector += 32 * kUnroll) {
      uint4 w[kRowsPerWarp][kUnroll];
#pragma unroll
      for (int item = 0; item < kRowsPerWarp; ++item) {
#pragma unroll
        for (int step = 0; step < kUnroll; ++step) {
          w[item][step] = load_streaming(rows[item] + vector + 32 * step);
        }
      }
#pragma unroll
      for (int step = 0; step < kUnroll; ++step) {
        const uint4 xv = __ldg(x + vector + 32 * step);
#pragma unroll
        for (int item = 0; item < kRowsPerWarp; ++item) {
          sums[item] = dot8<T>(w[item][step], xv, sums[item]);
        }
      }
    }
    for (; vector < vectors; vector += 32) {
      const uint4 xv = __ldg(x + vector);
#pragma unroll
      for (int item = 0; item < kRowsPerWarp; ++item) {
        sums[item] = dot8<T>(load_streaming(rows[item] + vector), xv, sums[item]);
      }
    }
  } else {
    for (int column = lane; column < k; column += 32) {
      const float value = Convert<T>::one(input[column]);
#pragma unroll
      for (int item = 0; item < kRowsPerWarp; ++item) {
        const int row = min(first_row + item, n - 1);
        sums[item] =
            fmaf(value, Convert<T>::one(weight[static_cast<size_t>(row) * k + column]), sums[item]);
      }
    }
  }

#pragma unroll
  for (int item = 0; item < kRowsPerWarp; ++item) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      sums[item] += __shfl_xor_sync(0xffffffffu, sums[item], offset);
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int item = 0; item < kRowsPerWarp; ++item) {
      const int row = first_row + item;
      if (row < n) {
        float result = alpha * sums[item];
        if (beta != 0.0f) result = fmaf(beta, Convert<T>::one(output[row]), result);
        output[row] = Convert<T>::from(result);
      }
    }
  }
}

template <typename T>
int launch(const Plan* plan, const void* input, const void* weight, void* output, float alpha,
           float beta) {
  const int rows_per_block = kWarps * kRowsPerWarp;
  const int blocks = (plan->n + rows_per_block - 1) / rows_per_block;
  dense_vector_kernel<T><<<blocks, kWarps * 32, 0, plan->stream>>>(
      static_cast<const T*>(input), static_cast<const T*>(weight), static_cast<T*>(output),
      plan->n, plan->k, alpha, beta);
  return static_cast<int>(cudaPeekAtLastError());
}

}  // namespace dense_vector
}  // namespace mircuda_b200

extern "C" int mircuda_dense_vector_create(int data_type, int n, int k, void* stream,
                                           void** output) {
  using namespace mircuda_b200::dense_vector;
  if ((data_type != 0 && data_type != 1) || n <= 0 || k <= 0 || stream == nullptr ||
      output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{data_type, n, k, static_cast<cudaStream_t>(stream)};
  if (plan == nullptr) return -2;
  *output = plan;
  return 0;
}

extern "C" int mircuda_dense_vector_execute(void* raw, void* stream, const void* input,
                                            const void* weight, void* output, float alpha,
                                            float beta) {
  using namespace mircuda_b200::dense_vector;
  if (raw == nullptr || stream == nullptr || input == nullptr || weight == nullptr ||
      output == nullptr) {
    return -1;
  }
  const auto* plan = static_cast<const Plan*>(raw);
  if (static_cast<cudaStream_t>(stream) != plan->stream) return -1;
  return plan->data_type == 0 ? launch<__half>(plan, input, weight, output, alpha, beta)
                              : launch<__nv_bfloat16>(plan, input, weight, output, alpha, beta);
}

extern "C" void mircuda_dense_vector_destroy(void* raw) {
  delete static_cast<mircuda_b200::dense_vector::Plan*>(raw);
}
