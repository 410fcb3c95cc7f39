// Block-scaled GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a:
//   C[M,N] (bf16) = alpha * A[M,K] . B[N,K]^T, fp32 accumulation in tensor memory,
// for MXFP8 (E4M3 codes, one UE8M0 scale per 32 K-elements, kind::mxf8f6f4) and NVFP4
// (E2M1 codes two per byte, one UE4M3 scale per 16, kind::mxf4nvf4 block16).
//
// Two CTAs on neighbouring SMs share one 256-row x BN-column output tile. Each CTA stages
// its own 128 rows of A and only HALF of the B tile (BN/2 rows) per 128-byte K stage; the
// MMA issued by the even ("leader") CTA reads both halves, so every operand byte crosses a
// shared-memory port once as a TMA write and once as an MMA read at half the rate of an
// unpaired CTA. That port, not HBM, is what bounds the unpaired kernel.
//
// Per CTA (192 threads): warp 0 = TMA producer (A, B-half, its A-scale atoms and all B-scale
// atoms of the tile, through tensor maps; completion bytes are counted on the LEADER's
// mbarrier), warp 1 = MMA issuer (leader only: tcgen05.cp of scale atoms to tensor memory of
// both CTAs, four MMAs per stage, commits that arrive on both CTAs' barriers), warps 2-5 =
// epilogue of the CTA's own 128 accumulator rows. No load replicates data to both CTAs.
// All mbarrier waits are bounded; the cluster barriers at start and end are reached by every
// thread on every path.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "launch_overlap.hpp"
#include "ptx.cuh"
#include "ptx_pair.cuh"
#include "tensor_map.hpp"

namespace mircuda_b200 {
namespace pair_gemm {

enum class Format { kMxFp8, kNvFp4 };

constexpr uint32_t kBlockM = 128;          // rows per CTA; the pair covers 256
constexpr uint32_t kStageBytesK = 128;     // bytes of K per stage row (128 E4M3 or 256 E2M1)
constexpr uint32_t kThreads = 192;
constexpr uint32_t kAtomBytes = 512;
constexpr uint32_t kTmemColumns = 512;

template <Format F>
struct FormatTraits;

template <>
struct FormatTraits<Format::kMxFp8> {
  static constexpr uint32_t kAtomsK = 1;            // scale atoms along K per stage
  static constexpr uint32_t kElementsPerStage = 128;
  static constexpr uint32_t kElementsPerAtom = 128; // 4 scale columns x 32
};

template <>
struct FormatTraits<Format::kNvFp4> {
  static constexpr uint32_t kAtomsK = 4;
  static constexpr uint32_t kElementsPerStage = 256;
  static constexpr uint32_t kElementsPerAtom = 64;  // 4 scale columns x 16
};

template <Format F, uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
struct Layout {
  // Multiples of 64 only: a tile then starts 0 or 2 columns into its first scale block in
  // tensor memory; an odd column offset is rejected by the MMA as a misaligned address.
  static_assert(BN == 128 || BN == 192 || BN == 256, "supported tile widths");
  using T = FormatTraits<F>;
  // Scale row tiles (128 rows) a BN-wide tile can touch, for every start offset it can have.
  static constexpr uint32_t kAtomsN = BN == 128 ? 1 : 2;
  static constexpr uint32_t kABytes = kBlockM * kStageBytesK;
  static constexpr uint32_t kBBytes = (BN / 2) * kStageBytesK;
  static constexpr uint32_t kSfaBytes = T::kAtomsK * kAtomBytes;
  static constexpr uint32_t kSfbBytes = kAtomsN * T::kAtomsK * kAtomBytes;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr uint32_t kBOffset = STAGES * kABytes;
  static constexpr uint32_t kSfaOffset = kBOffset + STAGES * kBBytes;
  static constexpr uint32_t kSfbOffset = kSfaOffset + STAGES * kSfaBytes;
  static constexpr uint32_t kBarrierOffset = kSfbOffset + STAGES * kSfbBytes;
  static constexpr uint32_t kBarriers = 2 * STAGES + 2 * ACC_STAGES;
  static constexpr uint32_t kMiscOffset = kBarrierOffset + kBarriers * 8;
  // Epilogue transpose buffers: 32 rows x 128 bytes for each of the four epilogue warps.
  static constexpr uint32_t kStagingOffset = (kMiscOffset + 16 + 127) / 128 * 128;
  static constexpr uint32_t kDynamicBytes = kStagingOffset + 4 * 4096 + 1024;
  // Tensor memory: accumulators, then as many scale buffers as fit (at most one per stage).
  // With several buffers the copy of the next stage's scales never has to wait for the
  // MMAs that still read the previous stage's.
  static constexpr uint32_t kSfColumns = 4 * T::kAtomsK * (1 + kAtomsN);   // per buffer
  static constexpr uint32_t kSfBuffersFit = (kTmemColumns - ACC_STAGES * BN) / kSfColumns;
  static constexpr uint32_t kSfBuffers = kSfBuffersFit < STAGES ? kSfBuffersFit : STAGES;
  static constexpr uint32_t kSfaColumn = ACC_STAGES * BN;                  // of buffer 0
  static constexpr uint32_t kSfbColumn = kSfaColumn + 4 * T::kAtomsK;
  static_assert(kSfBuffers >= 1, "tensor memory budget");
  static_assert(kBBytes % 1024 == 0, "B half must keep the 1024-byte swizzle period");
  static_assert(kDynamicBytes <= 232448, "shared memory budget");
};

// Fused GEMM + all-gather for column-sharded linears: when `count` is non-zero the epilogue
// does not write C[M, n] locally but stores every tile into the full-width output
// [M, row_stride] of each of `count` GPUs (this GPU's own buffer among them) at column
// `column_offset`, with ordinary stores through peer-mapped pointers or, when the buffers are
// bound to an NVSwitch multicast object, with one multimem store that the switch replicates.
// The transfer over NVLink then overlaps the MMAs of the following tiles and no separate
// collective runs.
struct Gather {
  __nv_bfloat16* outputs[8];
  // When not null: the multicast address of the same buffers (one NVSwitch multicast object
  // bound on every GPU). A single multimem store then reaches all of them, so this GPU's
  // NVLink egress is one copy of its shard instead of one per peer.
  __nv_bfloat16* multicast;
  uint32_t count;
  uint32_t row_stride;
  uint32_t column_offset;
};

struct Maps {
  CUtensorMap a;     // [M, K bytes], box 128 rows x 128 bytes, 128-byte swizzle
  CUtensorMap b;      // [N, K bytes], box BN/2 rows x 128 bytes
  CUtensorMap sfa;    // scales as u32 [row tiles][K atoms][128 words], box {128, atomsK, 1}
  CUtensorMap sfb;    // same for B, box {128, atomsK, atomsN}
};

template <Format F, uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
block_scaled_pair_gemm_kernel(const __grid_constant__ Maps maps, __nv_bfloat16* __restrict__ c,
                              uint32_t m, uint32_t n, uint32_t k_stages, float alpha,
                              uint32_t* __restrict__ status, const Gather gather) {
  using L = Layout<F, BN, STAGES, ACC_STAGES>;
  using T = FormatTraits<F>;
  extern __shared__ uint8_t dynamic_shared[];
  const uint32_t misalignment = ptx::smem_address(dynamic_shared) & 1023u;
  uint8_t* shared = dynamic_shared + ((1024u - misalignment) & 1023u);
  uint8_t* shared_a = shared;
  uint8_t* shared_b = shared + L::kBOffset;
  uint8_t* shared_sfa = shared + L::kSfaOffset;
  uint8_t* shared_sfb = shared + L::kSfbOffset;
  uint64_t* full = reinterpret_cast<uint64_t*>(shared + L::kBarrierOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(shared + L::kMiscOffset);
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const uint32_t warp = threadIdx.x / 32u;
  const uint32_t lane = threadIdx.x % 32u;
  const uint32_t rank = ptx::cluster_cta_rank();   // 0 = leader
  const bool leader = rank == 0u;

  if (threadIdx.x == 0) {
    for (uint32_t stage = 0; stage < STAGES; ++stage) {
      ptx::mbarrier_init(&full[stage], 2);          // one arrive.expect_tx per CTA
      ptx::mbarrier_init(&empty[stage], 1);         // one commit arrival
    }
    for (uint32_t stage = 0; stage < ACC_STAGES; ++stage) {
      ptx::mbarrier_init(&acc_full[stage], 1);
      ptx::mbarrier_init(&acc_empty[stage], 8);     // four epilogue warps in each CTA
    }
    *abort = 0u;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensor_map(&maps.a);
    ptx::prefetch_tensor_map(&maps.b);
    ptx::prefetch_tensor_map(&maps.sfa);
    ptx::prefetch_tensor_map(&maps.sfb);
  }
  if (warp == 1) {
    ptx::tmem_allocate_pair(tmem_slot, kTmemColumns);
    ptx::tmem_relinquish_pair();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched no global memory and may have run beside the tail of the kernel
  // before this one on the stream (the activation quantizer, normally); what follows may not.
  ptx::dependency_launch_next();
  ptx::dependency_wait();

  const uint32_t tiles_m = (m + 2u * kBlockM - 1u) / (2u * kBlockM);
  const uint32_t tiles_n = (n + BN - 1u) / BN;
  const uint32_t tiles = tiles_m * tiles_n;
  const uint32_t pair = blockIdx.x / 2u;
  const uint32_t pairs = gridDim.x / 2u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool running = true;
      for (uint32_t tile = pair; running && tile < tiles; tile += pairs) {
        const uint32_t m0 = (tile % tiles_m) * 2u * kBlockM + rank * kBlockM;
        const uint32_t n0 = (tile / tiles_m) * BN;
        for (uint32_t ks = 0; ks < k_stages; ++ks) {
          if (!ptx::mbarrier_wait_cluster(&empty[stage], phase ^ 1u, abort)) {
            running = false;
            break;
          }
          // Every byte this CTA loads is counted on the leader's barrier of this stage.
          const uint32_t barrier = ptx::map_to_cta(ptx::smem_address(&full[stage]), 0u);
          ptx::mbarrier_arrive_expect_tx_cluster(barrier, L::kStageBytes);
          const int32_t x = static_cast<int32_t>(ks * kStageBytesK);
          ptx::tma_load_2d_pair(shared_a + stage * L::kABytes, &maps.a, barrier, x,
                                static_cast<int32_t>(m0));
          ptx::tma_load_2d_pair(shared_b + stage * L::kBBytes, &maps.b, barrier, x,
                                static_cast<int32_t>(n0 + rank * (BN / 2u)));
          ptx::tma_load_3d_pair(shared_sfa + stage * L::kSfaBytes, &maps.sfa, barrier, 0,
                                static_cast<int32_t>(ks * T::kAtomsK),
                                static_cast<int32_t>(m0 / 128u));
          ptx::tma_load_3d_pair(shared_sfb + stage * L::kSfbBytes, &maps.sfb, barrier, 0,
                                static_cast<int32_t>(ks * T::kAtomsK),
                                static_cast<int32_t>(n0 / 128u));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort != 0u) {
        for (int spin = 0; spin < 256; ++spin) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------- MMA issuer (leader CTA only)
    if (leader && ptx::elect_one()) {
      constexpr uint32_t idesc =
          F == Format::kMxFp8
              ? ptx::make_block_scaled_idesc(ptx::kFormatE4M3, ptx::kFormatE4M3, 2u * kBlockM, BN, true)
              : ptx::make_block_scaled_idesc(ptx::kFormatE2M1_mxf4, ptx::kFormatE2M1_mxf4,
                                             2u * kBlockM, BN, false);
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0, sf_buffer = 0;
      bool running = true;
      for (uint32_t tile = pair; running && tile < tiles; tile += pairs) {
        const uint32_t n0 = (tile / tiles_m) * BN;
        const uint32_t sfb_shift = (n0 % 128u) / 32u;   // tile start inside its first scale atom
        if (!ptx::mbarrier_wait_cluster(&acc_empty[acc_stage], acc_phase ^ 1u, abort)) break;
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * BN;
        for (uint32_t ks = 0; ks < k_stages; ++ks) {
          if (!ptx::mbarrier_wait_cluster(&full[stage], phase, abort)) {
            running = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t sfa_tmem = tmem_base + L::kSfaColumn + sf_buffer * L::kSfColumns;
          const uint32_t sfb_tmem = tmem_base + L::kSfbColumn + sf_buffer * L::kSfColumns;
          if (++sf_buffer == L::kSfBuffers) sf_buffer = 0;
#pragma unroll
          for (uint32_t ka = 0; ka < T::kAtomsK; ++ka) {
            ptx::tcgen05_copy_scales_pair(
                sfa_tmem + 4u * ka,
                ptx::make_scale_descriptor(
                    ptx::smem_address(shared_sfa + stage * L::kSfaBytes + ka * kAtomBytes)));
#pragma unroll
            for (uint32_t atom = 0; atom < L::kAtomsN; ++atom) {
              ptx::tcgen05_copy_scales_pair(
                  sfb_tmem + 4u * (ka * L::kAtomsN + atom),
                  ptx::make_scale_descriptor(ptx::smem_address(
                      shared_sfb + stage * L::kSfbBytes + (atom * T::kAtomsK + ka) * kAtomBytes)));
            }
          }
          const uint64_t a_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_a + stage * L::kABytes));
          const uint64_t b_descriptor =
              ptx::make_k_major_sw128_descriptor(ptx::smem_address(shared_b + stage * L::kBBytes));
#pragma unroll
          for (uint32_t kb = 0; kb < 4u; ++kb) {
            const bool accumulate = (ks | kb) != 0u;
            if constexpr (F == Format::kMxFp8) {
              ptx::mma_mxf8f6f4_block_scale_pair(
                  d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb,
                  ptx::with_scale_ids(idesc, kb, kb), sfa_tmem, sfb_tmem + sfb_shift, accumulate);
            } else {
              ptx::mma_nvf4_block16_pair(
                  d_tmem, a_descriptor + 2u * kb, b_descriptor + 2u * kb, idesc,
                  sfa_tmem + 4u * kb, sfb_tmem + 4u * kb * L::kAtomsN + sfb_shift, accumulate);
            }
          }
          ptx::tcgen05_commit_pair(&empty[stage], 3u);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!running) break;
        ptx::tcgen05_commit_pair(&acc_full[acc_stage], 3u);
        if (++acc_stage == ACC_STAGES) {
          acc_stage = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------------- epilogue
    const uint32_t quarter = warp % 4u;
    const bool vector_stores = (n % 8u) == 0u;
    uint8_t* staging = shared + L::kStagingOffset + quarter * 4096u;
    uint32_t acc_stage = 0, acc_phase = 0;
    for (uint32_t tile = pair; tile < tiles; tile += pairs) {
      const uint32_t m0 = (tile % tiles_m) * 2u * kBlockM + rank * kBlockM;
      const uint32_t n0 = (tile / tiles_m) * BN;
      if (!ptx::mbarrier_wait_cluster(&acc_full[acc_stage], acc_phase, abort)) break;
      ptx::tcgen05_fence_after();
      const uint32_t row = m0 + quarter * 32u + lane;
      const uint32_t tmem_row = tmem_base + ((quarter * 32u) << 16) + acc_stage * BN;
#pragma unroll 1
      for (uint32_t chunk = 0; chunk < BN / 32u; ++chunk) {
        uint32_t values[32];
        ptx::tmem_load_32x32(tmem_row + chunk * 32u, values);
        ptx::tmem_load_wait();
        if (chunk + 1u == BN / 32u) {
          // Everything is in registers: hand the accumulator back before the stores go out.
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            ptx::mbarrier_arrive_cluster(ptx::map_to_cta(ptx::smem_address(&acc_empty[acc_stage]), 0u));
          }
        }
        const uint32_t column = n0 + chunk * 32u;
        if (vector_stores) {
          // A lane owns one accumulator row, so storing from registers would scatter 16-byte
          // pieces over 32 rows. The warp instead transposes 64 columns through shared memory
          // (16-byte pieces XOR-swizzled by row: conflict-free both ways) and writes whole
          // 128-byte row segments, eight lanes to a row. Over NVLink that is the difference
          // between 16-byte and 128-byte write packets.
#pragma unroll
          for (uint32_t part = 0; part < 4u; ++part) {
            uint32_t words[4];
#pragma unroll
            for (uint32_t pair_index = 0; pair_index < 4u; ++pair_index) {
              const __nv_bfloat162 two = __floats2bfloat162_rn(
                  __uint_as_float(values[part * 8u + pair_index * 2u]) * alpha,
                  __uint_as_float(values[part * 8u + pair_index * 2u + 1u]) * alpha);
              words[pair_index] = *reinterpret_cast<const uint32_t*>(&two);
            }
            const uint32_t piece = (chunk & 1u) * 4u + part;
            *reinterpret_cast<uint4*>(staging + lane * 128u + ((piece ^ (lane & 7u)) * 16u)) =
                make_uint4(words[0], words[1], words[2], words[3]);
          }
          if ((chunk & 1u) != 0u) {
            __syncwarp();
            const uint32_t piece = lane % 8u;
            const uint32_t piece_column = column - 32u + piece * 8u;
#pragma unroll
            for (uint32_t step = 0; step < 8u; ++step) {
              const uint32_t local_row = step * 4u + lane / 8u;
              const uint4 packed = *reinterpret_cast<const uint4*>(
                  staging + local_row * 128u + ((piece ^ (local_row & 7u)) * 16u));
              const uint32_t global_row = m0 + quarter * 32u + local_row;
              if (global_row < m && piece_column < n) {
                if (gather.count != 0u) {
                  // Fused all-gather: the same bytes go to every GPU's full-width output.
                  const size_t offset = static_cast<size_t>(global_row) * gather.row_stride +
                                        gather.column_offset + piece_column;
                  if (gather.multicast != nullptr) {
                    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(
                                     gather.multicast + offset),
                                 "r"(packed.x), "r"(packed.y), "r"(packed.z), "r"(packed.w)
                                 : "memory");
                  } else {
                    for (uint32_t target = 0; target < gather.count; ++target) {
                      *reinterpret_cast<uint4*>(gather.outputs[target] + offset) = packed;
                    }
                  }
                } else {
                  *reinterpret_cast<uint4*>(c + static_cast<size_t>(global_row) * n + piece_column) =
                      packed;
                }
              }
            }
            __syncwarp();
          }
        } else if (row < m && column < n) {
          __nv_bfloat16* destination = c + static_cast<size_t>(row) * n + column;
#pragma unroll
          for (uint32_t item = 0; item < 32u; ++item) {
            if (column + item < n) {
              destination[item] = __float2bfloat16_rn(__uint_as_float(values[item]) * alpha);
            }
          }
        }
      }
      if (++acc_stage == ACC_STAGES) {
        acc_stage = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // Neither CTA may free tensor memory or exit while the other can still signal its barriers
  // or while the leader's MMAs still read its shared memory.
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    __syncwarp();
    ptx::tcgen05_fence_after();
    ptx::tmem_deallocate_pair(tmem_base, kTmemColumns);
  }
  if (threadIdx.x == 0 && *abort != 0u) *status = 1u;
}

// ------------------------------------------------------------------------------- host

// Scales viewed as u32 [row tiles][K atoms][128 words]; one box = whole 512-byte atoms.
inline int encode_scale_map(CUtensorMap* map, const void* base, uint64_t row_tiles,
                            uint64_t k_atoms, uint32_t box_k_atoms, uint32_t box_row_tiles) {
  EncodeTiled encode = encode_tiled_entry();
  if (encode == nullptr) return static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dimensions[3] = {128u, k_atoms, row_tiles};
  const cuuint64_t strides[2] = {kAtomBytes, k_atoms * kAtomBytes};
  const cuuint32_t box[3] = {128u, box_k_atoms, box_row_tiles};
  const cuuint32_t element_strides[3] = {1u, 1u, 1u};
  return static_cast<int>(encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3u, const_cast<void*>(base),
                                 dimensions, strides, box, element_strides,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
}

struct Problem {
  uint32_t m, n, k;          // k in elements
  int device, sm_count;
  cudaStream_t stream;
  uint32_t* status;
};

// Encodes the four tensor maps for the given operand pointers.
template <Format F>
int encode_maps(Maps* maps, const Problem& problem, uint32_t block_n, const void* a,
                const void* a_scales, const void* b, const void* b_scales) {
  using T = FormatTraits<F>;
  const uint64_t k_bytes = F == Format::kMxFp8 ? problem.k : problem.k / 2u;
  const uint64_t k_atoms = problem.k / T::kElementsPerAtom;
  const uint32_t atoms_n = block_n == 128u ? 1u : 2u;
  int status = encode_k_major_map(&maps->a, a, problem.m, k_bytes, 1u, kBlockM);
  if (status == 0) status = encode_k_major_map(&maps->b, b, problem.n, k_bytes, 1u, block_n / 2u);
  if (status == 0) {
    status = encode_scale_map(&maps->sfa, a_scales, (problem.m + 127u) / 128u, k_atoms, T::kAtomsK, 1u);
  }
  if (status == 0) {
    status = encode_scale_map(&maps->sfb, b_scales, (problem.n + 127u) / 128u, k_atoms, T::kAtomsK,
                              atoms_n);
  }
  return status;
}

template <Format F, uint32_t BN, uint32_t STAGES, uint32_t ACC_STAGES>
int launch(const Problem& problem, const Maps& maps, void* c, float alpha,
           const Gather& gather = Gather{}) {
  using L = Layout<F, BN, STAGES, ACC_STAGES>;
  using T = FormatTraits<F>;
  auto function = block_scaled_pair_gemm_kernel<F, BN, STAGES, ACC_STAGES>;
  static thread_local int configured_device = -1;
  static thread_local int resident_pairs = 0;
  if (configured_device != problem.device) {
    int status = static_cast<int>(cudaFuncSetAttribute(
        function, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
    if (status != 0) return status;
    // The kernel is persistent: every pair must be resident at once, or the pairs that are
    // not would only start after a resident one has finished all its tiles. Not every SM
    // can be paired (it depends on how SMs are grouped on the die), so ask.
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned int>(problem.sm_count) & ~1u, 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = L::kDynamicBytes;
    cudaLaunchAttribute attribute = {};
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    status = static_cast<int>(cudaOccupancyMaxActiveClusters(&clusters, function, &config));
    if (status != 0) return status;
    if (clusters < 1) return static_cast<int>(cudaErrorLaunchOutOfResources);
    resident_pairs = clusters;
    configured_device = problem.device;
    if (std::getenv("MIRCUDA_B200_DEBUG") != nullptr) {
      std::fprintf(stderr, "mircuda_b200: %d resident CTA pairs on %d SMs (BN=%u)\n", clusters,
                   problem.sm_count, BN);
    }
  }
  const uint32_t tiles = ((problem.m + 255u) / 256u) * ((problem.n + BN - 1u) / BN);
  uint32_t pairs = static_cast<uint32_t>(resident_pairs);
  if (tiles < pairs) pairs = tiles;
  const uint32_t k_stages = (problem.k + T::kElementsPerStage - 1u) / T::kElementsPerStage;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2u * pairs, 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = L::kDynamicBytes;
  config.stream = problem.stream;
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = overlap_launches() ? 1u : 0u;
  return static_cast<int>(cudaLaunchKernelEx(&config, function, maps, static_cast<__nv_bfloat16*>(c),
                                             problem.m, problem.n, k_stages, alpha, problem.status,
                                             gather));
}

}  // namespace pair_gemm
}  // namespace mircuda_b200
