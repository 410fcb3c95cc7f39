// W4A16 with symmetric int4 weights: y[m, n] = f16(sum_k x[m, k] * (q[n, k] - 8) * s[n, k / 128]),
// f16 activations and outputs, fp32 accumulation. Weights are [N, K/2] bytes, two codes per
// byte (even k in the low nibble), q in 0..15 standing for q - 8; scales are f16 [N, K/128].
// The reference has no int4 entry point (its W4A16 is the NVFP4/MXFP4 Marlin path); this op
// covers the int4-g128 decode/prefill shapes: exact q - 8 in f16, f16 tensor-core products,
// fp32 accumulation.
//
// M <= 16 is bound by HBM (the weights are read once): a CTA owns 128 weight rows and a part
// of K; a producer warp streams 512-element stages (one [128 x 256 B] TMA box) through a
// two-stage ring; eight consumer warps dequantise with the magic-number trick (a nibble OR-ed
// into the mantissa of 1024.0 is 1024 + q; one exact packed subtract or FMA gives q - 8), 1.1
// instructions per weight, and feed mma.sync.m16n8k16 with the weights on the 16-row side and
// the tokens on the 8-wide side (one or two token groups); a warp's 128 K-elements of a stage
// are one scale group, so the scale multiplies the group's fp32 sum once. The K parts of a
// row tile form a thread-block cluster and meet in the first CTA's shared memory (DSMEM).
// M > 16 is bound by the tensor cores: the weights are expanded once to f16 in a workspace the
// plan owns and multiplied by the tcgen05 dense GEMM (dense_gemm.cu).
// Every mbarrier wait is bounded; the cluster barrier is reached on every path.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>

#include "ptx.cuh"
#include "ptx_pair.cuh"
#include "tensor_map.hpp"
#include "w4a16_stream.hpp"
#include "w4a16_tile.hpp"

extern "C" int mircuda_dense_create(int input_type, int output_type, int m, int n, int k,
                                    void* stream, void** output);
extern "C" int mircuda_dense_execute(void* plan, void* stream, const void* a, const void* b,
                                     void* c, float alpha, float beta);
extern "C" void mircuda_dense_destroy(void* plan);

namespace mircuda_b200 {
namespace w4a16 {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;   // + one producer warp
constexpr int kTileRows = 128;
constexpr int kStageK = 512;
constexpr int kStageBytes = kTileRows * kStageK / 2;  // 32 KB
constexpr int kStages = 2;
constexpr int kWarpsK = kStageK / 128;
constexpr int kRowGroups = kConsumerWarps / kWarpsK;
constexpr int kRowsPerWarp = kTileRows / kRowGroups;
constexpr int kSteps = kRowsPerWarp / 16;
constexpr int kGroupK = 128;
constexpr int kVectorTokens = 16;

template <int TG>
struct SharedLayout {
  static constexpr int kTokens = 8 * TG;
  static constexpr int kMaxParts = 8 / TG;
  static constexpr int kWeights = 0;
  static constexpr int kSums = 0;      // [kWarpsK][128][kTokens] f32, reuses the ring
  static constexpr int kParts = kStages * kStageBytes;           // [kMaxParts][128][kTokens] f32
  static constexpr int kBarriers = kParts + kMaxParts * kTileRows * kTokens * 4;
  static constexpr int kBytes = kBarriers + 2 * kStages * 8 + 16 + 1024;
  static_assert(kWarpsK * kTileRows * kTokens * 4 <= kStages * kStageBytes, "sums fit the ring");
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t bits) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(d) : "r"(a), "r"(mask), "r"(bits));   // (a & b) | c
  return d;
}

__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

__device__ __forceinline__ void mma_f16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1,
                                                uint32_t a2, uint32_t a3, uint32_t b0,
                                                uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Eight codes of one u32 (k0..k7, k0 lowest) -> (k0,k4) (k1,k5) (k2,k6) (k3,k7) as q - 8 in
// f16x2, exactly: 1024 + q minus 1032, and (1024 + 16 q) / 16 minus 72. The scale is applied
// later, in fp32, to the sum over the 128-element scale group (multiplying here by a rounded
// -1032 * s would cancel catastrophically).
__device__ __forceinline__ void dequantize8(uint32_t codes, uint32_t (&out)[4]) {
  const uint32_t shifted = codes >> 8;
  out[0] = sub_f16x2(lop3_and_or(codes, 0x000f000fu, 0x64006400u), 0x64086408u);
  out[1] = fma_f16x2(lop3_and_or(codes, 0x00f000f0u, 0x64006400u), 0x2c002c00u, 0xd480d480u);
  out[2] = sub_f16x2(lop3_and_or(shifted, 0x000f000fu, 0x64006400u), 0x64086408u);
  out[3] = fma_f16x2(lop3_and_or(shifted, 0x00f000f0u, 0x64006400u), 0x2c002c00u, 0xd480d480u);
}

template <int TG>
__global__ void __launch_bounds__(kThreads)
w4a16_vector_kernel(const __grid_constant__ CUtensorMap weight_map, const __half* __restrict__ input,
                    const __half* __restrict__ scales, __half* __restrict__ output, int m, int n,
                    int k, int parts, uint32_t* __restrict__ status) {
  using S = SharedLayout<TG>;
  constexpr int kTokens = S::kTokens;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_weights = shared + S::kWeights;
  float* shared_sums = reinterpret_cast<float*>(shared + S::kSums);
  float* shared_parts = reinterpret_cast<float*>(shared + S::kParts);
  uint64_t* full = reinterpret_cast<uint64_t*>(shared + S::kBarriers);
  uint64_t* empty = full + kStages;
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(empty + kStages);

  const int row_tile = blockIdx.x;
  const int part = blockIdx.y;                       // == rank inside the cluster
  const int stages_total = (k + kStageK - 1) / kStageK;
  const int stages_per_part = (stages_total + parts - 1) / parts;
  const int first_stage = part * stages_per_part;
  const int my_stages = max(0, min(stages_per_part, stages_total - first_stage));
  const int groups_k = k / kGroupK;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int stage = 0; stage < kStages; ++stage) {
      ptx::mbarrier_init(&full[stage], 1);
      ptx::mbarrier_init(&empty[stage], kConsumerWarps);
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&weight_map);
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // --------------------------------------------------------------------- producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      for (int index = 0; index < my_stages; ++index) {
        if (!ptx::mbarrier_wait(&empty[stage], phase ^ 1u, abort)) break;
        ptx::mbarrier_arrive_expect_tx(&full[stage], kStageBytes);
        ptx::tma_load_2d(shared_weights + stage * kStageBytes, &weight_map, &full[stage],
                         (first_stage + index) * (kStageK / 2), row_tile * kTileRows);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (*abort != 0u) {
        for (int spin = 0; spin < 256; ++spin) __nanosleep(1000);
      }
    }
  } else {
    // -------------------------------------------------------------------- consumers
    const int group = lane >> 2;                     // weight row inside a 16-row step / token
    const int quad = lane & 3;
    const int warp_k = warp % kWarpsK;               // 128-element K sub-range = one scale group
    const int warp_rows = warp / kWarpsK;
    const int chunk = warp_k * 4 + quad;             // this thread's 32-element chunk
    float accumulator[kSteps][TG][4];
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
#pragma unroll
      for (int tokens = 0; tokens < TG; ++tokens) {
#pragma unroll
        for (int item = 0; item < 4; ++item) accumulator[step][tokens][item] = 0.0f;
      }
    }
    uint32_t stage = 0, phase = 0;
    for (int index = 0; index < my_stages; ++index) {
      const int element = (first_stage + index) * kStageK + chunk * 32;
      const bool active = element < k;
      // B fragments (from L2, before the stage's arrival is awaited): token `group` of each
      // token group, 32 activations regrouped as (x0,x4) (x1,x5) (x2,x6) (x3,x7) per eight to
      // match the order the dequantisation produces.
      uint32_t b[TG][16];
#pragma unroll
      for (int tokens = 0; tokens < TG; ++tokens) {
        const int token = tokens * 8 + group;
        if (token < m && active) {
          const uint4* source = reinterpret_cast<const uint4*>(input + static_cast<size_t>(token) * k + element);
#pragma unroll
          for (int word = 0; word < 4; ++word) {
            const uint4 v = __ldg(source + word);
            b[tokens][word * 4 + 0] = prmt(v.x, v.z, 0x5410u);
            b[tokens][word * 4 + 1] = prmt(v.x, v.z, 0x7632u);
            b[tokens][word * 4 + 2] = prmt(v.y, v.w, 0x5410u);
            b[tokens][word * 4 + 3] = prmt(v.y, v.w, 0x7632u);
          }
        } else {
#pragma unroll
          for (int item = 0; item < 16; ++item) b[tokens][item] = 0u;
        }
      }
      // This stage's scales of the thread's rows: group element / 128 of rows (g, g + 8) of
      // every step. Rows past n and chunks past k get a zero scale (their codes are TMA fill).
      uint16_t scale_bits[kSteps][2];
#pragma unroll
      for (int step = 0; step < kSteps; ++step) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int row = row_tile * kTileRows + warp_rows * kRowsPerWarp + step * 16 + group + half * 8;
          scale_bits[step][half] = 0;
          if (active && row < n) {
            scale_bits[step][half] = __ldg(reinterpret_cast<const uint16_t*>(scales) +
                                           static_cast<size_t>(row) * groups_k + element / kGroupK);
          }
        }
      }
      if (!ptx::mbarrier_wait(&full[stage], phase, abort)) break;
      const uint8_t* weights = shared_weights + stage * kStageBytes;
#pragma unroll
      for (int step = 0; step < kSteps; ++step) {
        const int row_low = warp_rows * kRowsPerWarp + step * 16 + group;
        const int row_high = row_low + 8;
        const uint4 packed_low = *reinterpret_cast<const uint4*>(weights + row_low * (kStageK / 2) + chunk * 16);
        const uint4 packed_high = *reinterpret_cast<const uint4*>(weights + row_high * (kStageK / 2) + chunk * 16);
        const float scale_low = __half2float(__ushort_as_half(scale_bits[step][0]));
        const float scale_high = __half2float(__ushort_as_half(scale_bits[step][1]));
        // The warp's 128 K-elements of this stage are one scale group: unscaled integer
        // products are summed here and scaled once, in fp32.
        float partial[TG][4];
#pragma unroll
        for (int tokens = 0; tokens < TG; ++tokens) {
#pragma unroll
          for (int item = 0; item < 4; ++item) partial[tokens][item] = 0.0f;
        }
        const uint32_t words_low[4] = {packed_low.x, packed_low.y, packed_low.z, packed_low.w};
        const uint32_t words_high[4] = {packed_high.x, packed_high.y, packed_high.z, packed_high.w};
#pragma unroll
        for (int word = 0; word < 4; ++word) {
          uint32_t low[4], high[4];
          dequantize8(words_low[word], low);
          dequantize8(words_high[word], high);
#pragma unroll
          for (int pair = 0; pair < 2; ++pair) {
#pragma unroll
            for (int tokens = 0; tokens < TG; ++tokens) {
              mma_f16_16x8x16(partial[tokens], low[2 * pair], high[2 * pair],
                              low[2 * pair + 1], high[2 * pair + 1], b[tokens][word * 4 + 2 * pair],
                              b[tokens][word * 4 + 2 * pair + 1]);
            }
          }
        }
#pragma unroll
        for (int tokens = 0; tokens < TG; ++tokens) {
          accumulator[step][tokens][0] = fmaf(scale_low, partial[tokens][0], accumulator[step][tokens][0]);
          accumulator[step][tokens][1] = fmaf(scale_low, partial[tokens][1], accumulator[step][tokens][1]);
          accumulator[step][tokens][2] = fmaf(scale_high, partial[tokens][2], accumulator[step][tokens][2]);
          accumulator[step][tokens][3] = fmaf(scale_high, partial[tokens][3], accumulator[step][tokens][3]);
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbarrier_arrive(&empty[stage]);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    // All consumer warps are done with the ring before the sums overwrite it.
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
    // accumulator[step][t]: rows (group, group + 8) x tokens (8t + 2*quad, 8t + 2*quad + 1)
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
#pragma unroll
      for (int tokens = 0; tokens < TG; ++tokens) {
        const int row = warp_rows * kRowsPerWarp + step * 16 + group;
        float* base = shared_sums + (warp_k * kTileRows + row) * kTokens + tokens * 8 + 2 * quad;
        *reinterpret_cast<float2*>(base) =
            make_float2(accumulator[step][tokens][0], accumulator[step][tokens][1]);
        *reinterpret_cast<float2*>(base + 8 * kTokens) =
            make_float2(accumulator[step][tokens][2], accumulator[step][tokens][3]);
      }
    }
  }
  __syncthreads();

  // CTA partial [128 rows][kTokens] = sum over the K sub-ranges; it goes to slot `part` of the
  // first CTA's `shared_parts` (its own shared memory when there is one part).
  const uint32_t slot_base = ptx::smem_address(shared_parts + part * kTileRows * kTokens);
  const uint32_t remote_base = parts > 1 ? ptx::map_to_cta(slot_base, 0u) : slot_base;
  for (int index = threadIdx.x; index < kTileRows * kTokens; index += kThreads) {
    float sum = shared_sums[index];
#pragma unroll
    for (int sub = 1; sub < kWarpsK; ++sub) sum += shared_sums[sub * kTileRows * kTokens + index];
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_base + index * 4), "f"(sum) : "memory");
  }
  if (parts > 1) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  if (part == 0) {
    for (int index = threadIdx.x; index < kTileRows * kTokens; index += kThreads) {
      const int row = row_tile * kTileRows + index / kTokens;
      const int token = index % kTokens;
      float total = 0.0f;
      for (int slot = 0; slot < parts; ++slot) total += shared_parts[slot * kTileRows * kTokens + index];
      if (row < n && token < m) output[static_cast<size_t>(token) * n + row] = __float2half_rn(total);
    }
  }
  if (threadIdx.x == 0 && *abort != 0u) *status = 1u;
}

// Expansion to f16 for the tensor-core path: one thread per eight weights.
__global__ void __launch_bounds__(256)
w4a16_dequantize_kernel(const uint32_t* __restrict__ weight, const __half* __restrict__ scales,
                        uint4* __restrict__ output, size_t words, uint32_t words_per_row,
                        uint32_t groups_k) {
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < words;
       index += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = index / words_per_row;
    const uint32_t word = static_cast<uint32_t>(index - row * words_per_row);
    const uint32_t codes = __ldg(weight + index);
    const float scale = __half2float(__ldg(scales + row * groups_k + word * 8u / kGroupK));
    uint32_t packed[4];
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
      const float low = (static_cast<float>((codes >> (8 * pair)) & 15u) - 8.0f) * scale;
      const float high = (static_cast<float>((codes >> (8 * pair + 4)) & 15u) - 8.0f) * scale;
      const __half2 two = __floats2half2_rn(low, high);
      packed[pair] = *reinterpret_cast<const uint32_t*>(&two);
    }
    output[index] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

struct Plan {
  int m, n, k;
  int parts, token_groups;
  int device;
  cudaStream_t stream;
  uint32_t* status;          // pinned
  const void* cached_weight;
  CUtensorMap weight_map;
  void* dense;               // tensor-core path: dense f16 plan and the expanded weights
  __half* expanded;
  bool stream_kernel;        // the persistent streaming kernel of w4a16_stream.cu
  bool overlap_launches;
  w4a16_stream::Config stream_config;
  bool tile_kernel;          // the fused prefill GEMM of w4a16_tile.cu
  w4a16_tile::Config tile_config;
  void* partial;             // its fp32 partial results when K is split
};

int parts_for(int n, int k, int slots, int max_parts) {
  const int row_tiles = (n + kTileRows - 1) / kTileRows;
  const int stages = (k + kStageK - 1) / kStageK;
  int best = 1;
  long long best_length = 0;
  for (int parts = 1; parts <= max_parts && parts <= stages; parts *= 2) {
    const int per_cta = (stages + parts - 1) / parts;
    const long long ctas = static_cast<long long>(row_tiles) * parts;
    const long long rounds = (ctas + slots - 1) / slots;
    const long long length = rounds * per_cta;
    if (parts == 1 || length < best_length) {
      best = parts;
      best_length = length;
    }
  }
  return best;
}

template <int TG>
int launch_vector(Plan* plan, const void* input, const void* scales, void* output) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((plan->n + kTileRows - 1) / kTileRows, plan->parts, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = SharedLayout<TG>::kBytes;
  config.stream = plan->stream;
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 1;
  attribute.val.clusterDim.y = plan->parts;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(
      &config, w4a16_vector_kernel<TG>, plan->weight_map, static_cast<const __half*>(input),
      static_cast<const __half*>(scales), static_cast<__half*>(output), plan->m, plan->n, plan->k,
      plan->parts, plan->status));
}

}  // namespace w4a16
}  // namespace mircuda_b200

extern "C" int mircuda_b200_w4a16_create(int m, int n, int k, void* stream, void** output) {
  using namespace mircuda_b200::w4a16;
  if (m <= 0 || n <= 0 || k <= 0 || k % kGroupK != 0 || n % 8 != 0 || stream == nullptr ||
      output == nullptr) {
    return -1;
  }
  auto* plan = new (std::nothrow) Plan{};
  if (plan == nullptr) return -2;
  plan->m = m;
  plan->n = n;
  plan->k = k;
  plan->stream = static_cast<cudaStream_t>(stream);
  int sm_count = 0;
  int status = static_cast<int>(cudaGetDevice(&plan->device));
  if (status == 0) {
    status = static_cast<int>(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, plan->device));
  }
  if (status == 0) {
    status = static_cast<int>(cudaHostAlloc(reinterpret_cast<void**>(&plan->status),
                                            sizeof(uint32_t), cudaHostAllocMapped));
  }
  if (status == 0) *plan->status = 0u;
  // Decode shapes the persistent streaming kernel covers (n % 16 == 0, k % 2048 == 0) run on it:
  // K=4096 x N=14336 at M=1 took 16.5 us on the ring kernel below. MIRCUDA_B200_W4A16=ring keeps
  // the ring kernel. Launches overlap as for mircuda_b200_nvfp4_vector_* (weights and scales are
  // fetched while earlier work of the stream may still run; MIRCUDA_B200_OVERLAP_LAUNCHES=0
  // serialises them).
  if (status == 0 && m <= kVectorTokens) {
    const char* choice = std::getenv("MIRCUDA_B200_W4A16");
    if (!(choice != nullptr && std::strcmp(choice, "ring") == 0)) {
      const int prepared = mircuda_b200::w4a16_stream::prepare(&plan->stream_config, m, n, k);
      if (prepared == 0) {
        plan->stream_kernel = true;
        const char* overlap = std::getenv("MIRCUDA_B200_OVERLAP_LAUNCHES");
        plan->overlap_launches = overlap == nullptr || overlap[0] == '1';
      } else if (prepared != -1) {
        status = prepared;
      }
    }
  }
  if (status == 0 && m <= kVectorTokens && !plan->stream_kernel) {
    plan->token_groups = m <= 8 ? 1 : 2;
    if (plan->token_groups == 1) {
      status = static_cast<int>(cudaFuncSetAttribute(w4a16_vector_kernel<1>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     SharedLayout<1>::kBytes));
      plan->parts = parts_for(n, k, 2 * sm_count, SharedLayout<1>::kMaxParts);
    } else {
      status = static_cast<int>(cudaFuncSetAttribute(w4a16_vector_kernel<2>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     SharedLayout<2>::kBytes));
      plan->parts = parts_for(n, k, sm_count, SharedLayout<2>::kMaxParts);
    }
  } else if (status == 0 && m > kVectorTokens) {
    // Prefill runs on the fused GEMM of w4a16_tile.cu (the packed weights are expanded inside the
    // kernel); MIRCUDA_B200_W4A16_PREFILL=expand keeps the two-launch form below (expansion into
    // an f16 workspace, then the dense GEMM), which is also the fallback.
    const char* choice = std::getenv("MIRCUDA_B200_W4A16_PREFILL");
    if (!(choice != nullptr && std::strcmp(choice, "expand") == 0) &&
        mircuda_b200::w4a16_tile::eligible(m, n, k)) {
      status = mircuda_b200::w4a16_tile::prepare(&plan->tile_config, m, n, k);
      plan->tile_kernel = status == 0;
      if (status == 0 && plan->tile_config.workspace_bytes != 0u) {
        status = static_cast<int>(cudaMallocAsync(&plan->partial, plan->tile_config.workspace_bytes, plan->stream));
      }
    }
  }
  if (status == 0 && m > kVectorTokens && !plan->tile_kernel) {
    status = mircuda_dense_create(0, 0, m, n, k, stream, &plan->dense);
    if (status == 0) {
      status = static_cast<int>(cudaMallocAsync(reinterpret_cast<void**>(&plan->expanded),
                                                static_cast<size_t>(n) * k * sizeof(__half),
                                                plan->stream));
    }
  }
  if (status != 0) {
    if (plan->dense != nullptr) mircuda_dense_destroy(plan->dense);
    if (plan->expanded != nullptr) cudaFreeAsync(plan->expanded, plan->stream);
    if (plan->partial != nullptr) cudaFreeAsync(plan->partial, plan->stream);
    if (plan->status != nullptr) cudaFreeHost(plan->status);
    delete plan;
    return status;
  }
  *output = plan;
  return 0;
}

extern "C" size_t mircuda_b200_w4a16_workspace_bytes(const void* raw) {
  const auto* plan = static_cast<const mircuda_b200::w4a16::Plan*>(raw);
  if (plan == nullptr) return 0;
  if (plan->tile_kernel) return plan->tile_config.workspace_bytes;
  if (plan->expanded == nullptr) return 0;
  return static_cast<size_t>(plan->n) * plan->k * sizeof(__half);
}

extern "C" int mircuda_b200_w4a16_execute(void* raw, void* stream, const void* input,
                                          const void* weight, const void* scales, void* output) {
  using namespace mircuda_b200;
  using namespace mircuda_b200::w4a16;
  if (raw == nullptr || stream == nullptr || input == nullptr || weight == nullptr ||
      scales == nullptr || output == nullptr) {
    return -1;
  }
  auto* plan = static_cast<Plan*>(raw);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  if (cuda_stream != plan->stream) return -1;
  if (*static_cast<volatile uint32_t*>(plan->status) != 0u) return -3;
  if (((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(input) |
        reinterpret_cast<uintptr_t>(output)) & 15u) != 0u ||
      (reinterpret_cast<uintptr_t>(scales) & 1u) != 0u) {
    return -1;
  }
  if (plan->stream_kernel) {
    if ((reinterpret_cast<uintptr_t>(scales) & 3u) != 0u) return -1;
    return mircuda_b200::w4a16_stream::launch(&plan->stream_config, cuda_stream, plan->overlap_launches, input, weight,
                                scales, output, plan->m, plan->n, plan->k, plan->status);
  }
  if (plan->tile_kernel) {
    return mircuda_b200::w4a16_tile::launch(&plan->tile_config, cuda_stream, input, weight, scales, output,
                                            plan->partial, plan->m, plan->n, plan->k, plan->status);
  }
  if (plan->dense != nullptr) {
    const size_t words = static_cast<size_t>(plan->n) * plan->k / 8u;
    const size_t blocks = (words + 255u) / 256u;
    w4a16_dequantize_kernel<<<static_cast<unsigned int>(blocks < 148u * 32u ? blocks : 148u * 32u), 256, 0,
                              cuda_stream>>>(
        static_cast<const uint32_t*>(weight), static_cast<const __half*>(scales),
        reinterpret_cast<uint4*>(plan->expanded), words, static_cast<uint32_t>(plan->k / 8),
        static_cast<uint32_t>(plan->k / kGroupK));
    const int status = static_cast<int>(cudaPeekAtLastError());
    if (status != 0) return status;
    return mircuda_dense_execute(plan->dense, stream, input, plan->expanded, output, 1.0f, 0.0f);
  }
  if (weight != plan->cached_weight) {
    EncodeTiled encode = encode_tiled_entry();
    if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
    const cuuint64_t dimensions[2] = {static_cast<cuuint64_t>(plan->k / 2), static_cast<cuuint64_t>(plan->n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(plan->k / 2)};
    const cuuint32_t box[2] = {kStageK / 2, kTileRows};
    const cuuint32_t element_strides[2] = {1u, 1u};
    const int status = static_cast<int>(encode(
        &plan->weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2u, const_cast<void*>(weight), dimensions,
        strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    if (status != 0) return status;
    plan->cached_weight = weight;
  }
  return plan->token_groups == 1 ? launch_vector<1>(plan, input, scales, output)
                                 : launch_vector<2>(plan, input, scales, output);
}

extern "C" void mircuda_b200_w4a16_destroy(void* raw) {
  auto* plan = static_cast<mircuda_b200::w4a16::Plan*>(raw);
  if (plan == nullptr) return;
  if (plan->dense != nullptr) mircuda_dense_destroy(plan->dense);
  if (plan->expanded != nullptr) cudaFreeAsync(plan->expanded, plan->stream);
  if (plan->partial != nullptr) cudaFreeAsync(plan->partial, plan->stream);
  if (plan->status != nullptr) cudaFreeHost(plan->status);
  delete plan;
}
