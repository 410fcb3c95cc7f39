// Row-wise helpers around the grouped MoE GEMMs (bandwidth-bound, bf16 rows, 16-byte
// accesses). They are the callers' side of the hot path: packing routed token rows into the
// compact per-expert layout the grouped plans read, the SwiGLU between the two expert GEMMs
// and the weighted sum of each token's expert outputs. The reference leaves these to its
// callers; there is no reference kernel to replace.
//   scatter_rows : dst[dst_index[i], :] = src[src_index[i], :]            i < count
//   swiglu       : out[r, j] = silu(in[r, j]) * in[r, I + j]              (in [rows, 2I])
//   combine_rows : out[t, :] = sum_j weight[t, j] * y[index[t, j], :]     fp32 accumulation
//   group_offsets: per-group row counts -> rows[] / offsets[] of the grouped plans, on the device
// and, for expert parallelism over NVLink peer memory (no collective kernel on the data path):
//   expert_layout: everyone's per-expert counts -> where this rank's rows go on each owner
//   dispatch_rows: token rows stored straight into the owners' receive buffers
//   collect_rows : each token's expert rows loaded from the owners' result buffers and summed
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "launch_overlap.hpp"
#include "ptx.cuh"

namespace mircuda_b200 {
namespace moe_rows {

constexpr int kThreads = 256;

// Every kernel here begins with a dependency wait and is launched with programmatic stream
// serialisation (launch_after_dependency): its CTAs may be scheduled while the kernel before it on
// the stream is finishing, but touch no global memory until that kernel has completed. A layer is
// a chain of a dozen launches of a few microseconds each; this takes the launch latency out of it.

__device__ __forceinline__ float2 unpack(uint32_t pair) {
  return make_float2(__uint_as_float(pair << 16), __uint_as_float(pair & 0xffff0000u));
}

__device__ __forceinline__ uint32_t pack(float low, float high) {
  const __nv_bfloat162 two = __floats2bfloat162_rn(low, high);
  return *reinterpret_cast<const uint32_t*>(&two);
}

// One warp per row copy; lanes stride over the row's 16-byte pieces.
__global__ void __launch_bounds__(kThreads)
moe_scatter_rows_kernel(const uint4* __restrict__ source, const int* __restrict__ source_index,
                        const int* __restrict__ destination_index, uint4* __restrict__ destination,
                        uint32_t count, uint32_t pieces) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  const uint32_t warps = gridDim.x * (kThreads / 32);
  const uint32_t lane = threadIdx.x % 32u;
  for (uint32_t item = blockIdx.x * (kThreads / 32) + threadIdx.x / 32u; item < count; item += warps) {
    const int from = __ldg(source_index + item);
    const int to = __ldg(destination_index + item);
    if (to < 0) continue;
    const uint4* in = source + static_cast<size_t>(from < 0 ? 0 : from) * pieces;
    uint4* out = destination + static_cast<size_t>(to) * pieces;
    for (uint32_t piece = lane; piece < pieces; piece += 32u) {
      out[piece] = from < 0 ? make_uint4(0u, 0u, 0u, 0u) : __ldg(in + piece);
    }
  }
}

__global__ void __launch_bounds__(kThreads)
moe_swiglu_kernel(const uint4* __restrict__ input, uint4* __restrict__ output, uint32_t rows,
                  const unsigned int* __restrict__ row_bound,
                  uint32_t pieces) {   // pieces = intermediate / 8
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  if (row_bound != nullptr) rows = min(rows, __ldg(row_bound));
  const size_t total = static_cast<size_t>(rows) * pieces;
  for (size_t item = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; item < total;
       item += static_cast<size_t>(gridDim.x) * kThreads) {
    const size_t row = item / pieces;
    const uint32_t piece = static_cast<uint32_t>(item - row * pieces);
    const uint4 gate = __ldg(input + row * 2u * pieces + piece);
    const uint4 up = __ldg(input + row * 2u * pieces + pieces + piece);
    const uint32_t gates[4] = {gate.x, gate.y, gate.z, gate.w};
    const uint32_t ups[4] = {up.x, up.y, up.z, up.w};
    uint32_t packed[4];
#pragma unroll
    for (int word = 0; word < 4; ++word) {
      const float2 g = unpack(gates[word]);
      const float2 u = unpack(ups[word]);
      packed[word] = pack(__fdividef(g.x, 1.0f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.0f + __expf(-g.y)) * u.y);
    }
    output[item] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

// One warp per token; each lane owns 16-byte pieces of the row and adds top_k rows in order.
__global__ void __launch_bounds__(kThreads)
moe_combine_rows_kernel(const uint4* __restrict__ rows, const int* __restrict__ index,
                        const float* __restrict__ weights, uint4* __restrict__ output,
                        uint32_t tokens, uint32_t top_k, uint32_t pieces) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  const uint32_t warps = gridDim.x * (kThreads / 32);
  const uint32_t lane = threadIdx.x % 32u;
  for (uint32_t token = blockIdx.x * (kThreads / 32) + threadIdx.x / 32u; token < tokens; token += warps) {
    for (uint32_t piece = lane; piece < pieces; piece += 32u) {
      float sums[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (uint32_t choice = 0; choice < top_k; ++choice) {
        const int row = __ldg(index + token * top_k + choice);
        if (row < 0) continue;
        const float weight = __ldg(weights + token * top_k + choice);
        const uint4 value = __ldg(rows + static_cast<size_t>(row) * pieces + piece);
        const uint32_t words[4] = {value.x, value.y, value.z, value.w};
#pragma unroll
        for (int word = 0; word < 4; ++word) {
          const float2 pair = unpack(words[word]);
          sums[2 * word] = fmaf(weight, pair.x, sums[2 * word]);
          sums[2 * word + 1] = fmaf(weight, pair.y, sums[2 * word + 1]);
        }
      }
      output[static_cast<size_t>(token) * pieces + piece] =
          make_uint4(pack(sums[0], sums[1]), pack(sums[2], sums[3]), pack(sums[4], sums[5]),
                     pack(sums[6], sums[7]));
    }
  }
}

// rows[g] = counts[g]; offsets[g] = block(g) * block_rows + aligned prefix of the counts before
// g inside its block of `per_block` groups. One thread per block of groups.
__global__ void moe_group_offsets_kernel(const int* __restrict__ counts, unsigned int* __restrict__ rows,
                                         unsigned int* __restrict__ offsets, uint32_t blocks,
                                         uint32_t per_block, uint32_t block_rows, uint32_t align) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  const uint32_t block = blockIdx.x * blockDim.x + threadIdx.x;
  if (block >= blocks) return;
  uint32_t cursor = block * block_rows;
  for (uint32_t item = 0; item < per_block; ++item) {
    const uint32_t group = block * per_block + item;
    const uint32_t count = static_cast<uint32_t>(max(counts[group], 0));
    rows[group] = count;
    offsets[group] = cursor;
    cursor += (count + align - 1u) / align * align;
  }
}

// Expert-parallel layout, one thread per global expert e (owner GPU = e / local_experts).
// all_counts[s][e] = rows GPU s routes to expert e. Every owner stores an expert's rows from
// all sources contiguously, sources in rank order, experts in index order:
//   start[e]        = rows of the owner's experts before e (each rounded up to `align` rows,
//                     128 to keep NVFP4 scale tiles per expert)
//   base_for_me[e]  = start[e] + rows of sources before `rank`  (where this rank's rows go)
//   rows/offsets    = the grouped plans' arrays for this rank's own experts
//   capacity_rows   = rows of every rank's receive buffer: an owner's rows / offsets are clamped
//                     to it (rows past it are neither dispatched nor computed) and `overflow`
//                     is raised on every rank that sees an expert run past it
__global__ void moe_expert_layout_kernel(const int* __restrict__ all_counts, uint32_t world,
                                         uint32_t rank, uint32_t experts, uint32_t local_experts,
                                         uint32_t align, int* __restrict__ base_for_me, unsigned int* __restrict__ rows,
                                         unsigned int* __restrict__ offsets,
                                         unsigned int* __restrict__ received_rows,
                                         uint32_t capacity_rows, unsigned int* __restrict__ overflow) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  extern __shared__ uint32_t totals[];
  const uint32_t expert = threadIdx.x;
  uint32_t total = 0u, before_me = 0u;
  if (expert < experts) {
    for (uint32_t source = 0; source < world; ++source) {
      const uint32_t count = static_cast<uint32_t>(max(all_counts[source * experts + expert], 0));
      if (source < rank) before_me += count;
      total += count;
    }
    totals[expert] = total;
  }
  __syncthreads();
  if (expert >= experts) return;
  const uint32_t owner_first = expert / local_experts * local_experts;
  uint32_t start = 0u;
  for (uint32_t other = owner_first; other < expert; ++other) {
    start += (totals[other] + align - 1u) / align * align;
  }
  base_for_me[expert] = static_cast<int>(start + before_me);
  if (start + total > capacity_rows && overflow != nullptr) *overflow = 1u;
  if (expert / local_experts == rank) {
    const uint32_t clamped_start = min(start, capacity_rows);
    rows[expert - owner_first] = min(total, capacity_rows - clamped_start);
    offsets[expert - owner_first] = clamped_start;
    if (expert - owner_first + 1u == local_experts && received_rows != nullptr) {
      *received_rows = min(start + (total + align - 1u) / align * align, capacity_rows);
    }
  }
}

struct PeerBases {
  void* base[8];
};

// Dispatch over peer memory: row i of this rank's expert-sorted assignments is copied from its
// token's activations straight into the owning GPU's receive buffer (ordinary stores through
// peer-mapped pointers, 512 contiguous bytes per warp instruction). The row index is kept for
// the way back.
__global__ void __launch_bounds__(kThreads)
moe_dispatch_rows_kernel(const uint4* __restrict__ source, const int* __restrict__ source_index,
                         const int* __restrict__ sorted_expert, const int* __restrict__ position,
                         const int* __restrict__ base_for_me, const PeerBases receive,
                         int* __restrict__ remote_row, uint32_t count, uint32_t local_experts,
                         uint32_t pieces, uint32_t capacity_rows) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  const uint32_t warps = gridDim.x * (kThreads / 32);
  const uint32_t lane = threadIdx.x % 32u;
  for (uint32_t item = blockIdx.x * (kThreads / 32) + threadIdx.x / 32u; item < count; item += warps) {
    const int expert = __ldg(sorted_expert + item);
    const uint32_t owner = static_cast<uint32_t>(expert) / local_experts;
    // An expert index outside the job (no such owner) is treated like a row that does not fit.
    const bool known = expert >= 0 && owner < 8u && receive.base[owner] != nullptr;
    const int row = known ? __ldg(base_for_me + expert) + __ldg(position + item) : -1;
    // A row at or past the owner's capacity is not sent (the layout kernel has raised the
    // overflow word and the owner computes nothing for it); -1 tells the way back to skip it.
    if (row < 0 || static_cast<uint32_t>(row) >= capacity_rows) {
      if (lane == 0) remote_row[item] = -1;
      continue;
    }
    if (lane == 0) remote_row[item] = row;
    const uint4* in = source + static_cast<size_t>(__ldg(source_index + item)) * pieces;
    uint4* out = static_cast<uint4*>(receive.base[owner]) + static_cast<size_t>(row) * pieces;
    for (uint32_t piece = lane; piece < pieces; piece += 32u) out[piece] = __ldg(in + piece);
  }
}

// Combine over peer memory: every token reads its top_k expert rows from the owners' output
// buffers (peer loads) and adds them with its routing weights. slot[t, j] is the position of
// (token, choice) in the expert-sorted assignment list.
// All top_k rows of a piece are requested before the first is used: their row indices and
// weights are read once per token (lane j holds choice j) and broadcast. A token's row is cut
// into `parts` runs of pieces, one warp each, so that a rank with few tokens (an 8-GPU job has
// 512) still has thousands of loads in flight.
template <int TOP_K>
__global__ void __launch_bounds__(kThreads)
moe_collect_rows_kernel(const PeerBases results, const int* __restrict__ slot,
                        const int* __restrict__ sorted_expert, const int* __restrict__ remote_row,
                        const float* __restrict__ weights, uint4* __restrict__ output,
                        uint32_t tokens, uint32_t top_k, uint32_t local_experts, uint32_t pieces,
                        uint32_t parts) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  const uint32_t warps = gridDim.x * (kThreads / 32);
  const uint32_t lane = threadIdx.x % 32u;
  const uint32_t part_pieces = (pieces + parts - 1u) / parts;
  for (uint32_t item = blockIdx.x * (kThreads / 32) + threadIdx.x / 32u; item < tokens * parts; item += warps) {
    const uint32_t token = item / parts;
    const uint32_t first_piece = (item % parts) * part_pieces;
    const uint32_t end_piece = min(pieces, first_piece + part_pieces);
    const uint4* my_row = nullptr;
    float my_weight = 0.0f;
    if (lane < top_k) {
      const int item = __ldg(slot + token * top_k + lane);
      if (item >= 0 && static_cast<uint32_t>(item) < tokens * top_k) {
        const uint32_t owner = static_cast<uint32_t>(__ldg(sorted_expert + item)) / local_experts;
        const int row = remote_row[item];
        // a row that did not fit the owner's buffer contributes nothing
        if (row >= 0 && owner < 8u && results.base[owner] != nullptr) {
          my_row = static_cast<const uint4*>(results.base[owner]) + static_cast<size_t>(row) * pieces;
          my_weight = __ldg(weights + token * top_k + lane);
        }
      }
    }
    // Every lane runs the same number of rounds (the shuffles below need the whole warp); lanes
    // past the end of the run load and store nothing.
    for (uint32_t round = first_piece; round < end_piece; round += 32u) {
      const uint32_t piece = round + lane;
      const bool active = piece < end_piece;
      uint4 values[TOP_K];
      float scale[TOP_K];
#pragma unroll
      for (int choice = 0; choice < TOP_K; ++choice) {
        const uint4* row = reinterpret_cast<const uint4*>(
            __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_row), choice));
        scale[choice] = __shfl_sync(0xffffffffu, my_weight, choice);
        values[choice] = (active && static_cast<uint32_t>(choice) < top_k && row != nullptr)
                             ? row[piece]
                             : make_uint4(0u, 0u, 0u, 0u);
      }
      float sums[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int choice = 0; choice < TOP_K; ++choice) {
        const uint32_t words[4] = {values[choice].x, values[choice].y, values[choice].z, values[choice].w};
#pragma unroll
        for (int word = 0; word < 4; ++word) {
          const float2 pair = unpack(words[word]);
          sums[2 * word] = fmaf(scale[choice], pair.x, sums[2 * word]);
          sums[2 * word + 1] = fmaf(scale[choice], pair.y, sums[2 * word + 1]);
        }
      }
      if (active) {
        output[static_cast<size_t>(token) * pieces + piece] =
            make_uint4(pack(sums[0], sums[1]), pack(sums[2], sums[3]), pack(sums[4], sums[5]),
                       pack(sums[6], sums[7]));
      }
    }
  }
}

// Row-major scale bytes [rows, columns] -> 512-byte atoms of 128 rows x 4 columns, 16 columns
// (four 4-byte atom pieces) per thread, only the first min(rows, *row_bound) rows.
__global__ void __launch_bounds__(kThreads)
moe_scale_atoms_kernel(const uint4* __restrict__ input, uint8_t* __restrict__ output, uint32_t rows,
                       const unsigned int* __restrict__ row_bound, uint32_t columns) {
  ptx::dependency_launch_next();
  ptx::dependency_wait();
  if (row_bound != nullptr) rows = min(rows, __ldg(row_bound));
  const uint32_t vectors = columns / 16u;
  const size_t total = static_cast<size_t>(rows) * vectors;
  const uint32_t column_tiles = columns / 4u;
  for (size_t item = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; item < total;
       item += static_cast<size_t>(gridDim.x) * kThreads) {
    const uint32_t row = static_cast<uint32_t>(item / vectors);
    const uint32_t vector = static_cast<uint32_t>(item - static_cast<size_t>(row) * vectors);
    const uint4 value = __ldg(input + item);
    const uint32_t words[4] = {value.x, value.y, value.z, value.w};
    uint8_t* base = output + (static_cast<size_t>(row / 128u) * column_tiles + vector * 4u) * 512u +
                    (row % 32u) * 16u + ((row % 128u) / 32u) * 4u;
#pragma unroll
    for (int tile = 0; tile < 4; ++tile) {
      *reinterpret_cast<uint32_t*>(base + tile * 512) = words[tile];
    }
  }
}

inline int grid_for(size_t work_items, int per_block) {
  const size_t blocks = (work_items + per_block - 1) / per_block;
  const size_t limit = 148u * 16u;     // enough CTAs to fill a B200 several times over
  return static_cast<int>(blocks < 1 ? 1 : (blocks > limit ? limit : blocks));
}

inline bool aligned16(const void* pointer) {
  return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0u;
}

}  // namespace moe_rows
}  // namespace mircuda_b200

extern "C" int mircuda_b200_moe_scatter_rows_bf16(const void* source, const int* source_index,
                                                  const int* destination_index, void* destination,
                                                  uint32_t count, uint32_t columns, void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (source == nullptr || source_index == nullptr || destination_index == nullptr ||
      destination == nullptr || columns == 0 || columns % 8 != 0 || !aligned16(source) ||
      !aligned16(destination)) {
    return -1;
  }
  if (count == 0) return 0;
  return mircuda_b200::launch_after_dependency(moe_scatter_rows_kernel, dim3(grid_for(count, kThreads / 32)), dim3(kThreads),
                                 0, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(source),
                                 source_index, destination_index, static_cast<uint4*>(destination), count,
                                 columns / 8u);
}

extern "C" int mircuda_b200_moe_swiglu_bf16(const void* input, void* output, uint32_t rows,
                                            const unsigned int* row_bound, uint32_t intermediate,
                                            void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (input == nullptr || output == nullptr || intermediate == 0 || intermediate % 8 != 0 ||
      !aligned16(input) || !aligned16(output)) {
    return -1;
  }
  if (rows == 0) return 0;
  const size_t total = static_cast<size_t>(rows) * (intermediate / 8u);
  return mircuda_b200::launch_after_dependency(moe_swiglu_kernel, dim3(grid_for(total, kThreads)), dim3(kThreads), 0,
                                 static_cast<cudaStream_t>(stream), static_cast<const uint4*>(input),
                                 static_cast<uint4*>(output), rows, row_bound, intermediate / 8u);
}

extern "C" int mircuda_b200_moe_combine_rows_bf16(const void* rows, const int* index,
                                                  const float* weights, void* output,
                                                  uint32_t tokens, uint32_t top_k, uint32_t columns,
                                                  void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (rows == nullptr || index == nullptr || weights == nullptr || output == nullptr ||
      top_k == 0 || columns == 0 || columns % 8 != 0 || !aligned16(rows) || !aligned16(output)) {
    return -1;
  }
  if (tokens == 0) return 0;
  return mircuda_b200::launch_after_dependency(moe_combine_rows_kernel, dim3(grid_for(tokens, kThreads / 32)), dim3(kThreads),
                                 0, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(rows), index,
                                 weights, static_cast<uint4*>(output), tokens, top_k, columns / 8u);
}

extern "C" int mircuda_b200_moe_group_offsets(const int* counts, unsigned int* rows,
                                              unsigned int* offsets, uint32_t blocks,
                                              uint32_t per_block, uint32_t block_rows,
                                              uint32_t align, void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (counts == nullptr || rows == nullptr || offsets == nullptr || blocks == 0 || per_block == 0 ||
      align == 0) {
    return -1;
  }
  return mircuda_b200::launch_after_dependency(moe_group_offsets_kernel, dim3((blocks + 63u) / 64u), dim3(64), 0,
                                 static_cast<cudaStream_t>(stream), counts, rows, offsets, blocks, per_block,
                                 block_rows, align);
}

extern "C" int mircuda_b200_moe_expert_layout(const int* all_counts, uint32_t world, uint32_t rank,
                                              uint32_t experts, uint32_t align, int* base_for_me,
                                              unsigned int* rows, unsigned int* offsets,
                                              unsigned int* received_rows, uint32_t capacity_rows,
                                              unsigned int* overflow, void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (all_counts == nullptr || base_for_me == nullptr || rows == nullptr || offsets == nullptr ||
      world == 0 || world > 8 || rank >= world || experts == 0 || experts > 1024 ||
      experts % world != 0 || align == 0 || capacity_rows == 0 || capacity_rows > 0x7fffffffu) {
    return -1;
  }
  return mircuda_b200::launch_after_dependency(moe_expert_layout_kernel, dim3(1), dim3(experts), experts * sizeof(uint32_t),
                                 static_cast<cudaStream_t>(stream), all_counts, world, rank, experts,
                                 experts / world, align, base_for_me, rows, offsets, received_rows, capacity_rows,
                                 overflow);
}

extern "C" int mircuda_b200_moe_dispatch_rows_bf16(
    const void* source, const int* source_index, const int* sorted_expert, const int* position,
    const int* base_for_me, void* const* receive_buffers, uint32_t world, int* remote_row,
    uint32_t count, uint32_t local_experts, uint32_t columns, uint32_t capacity_rows, void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (source == nullptr || source_index == nullptr || sorted_expert == nullptr ||
      position == nullptr || base_for_me == nullptr || receive_buffers == nullptr ||
      remote_row == nullptr || world == 0 || world > 8 || local_experts == 0 || columns == 0 ||
      columns % 8 != 0 || !aligned16(source) || capacity_rows == 0 || capacity_rows > 0x7fffffffu) {
    return -1;
  }
  PeerBases receive = {};
  for (uint32_t peer = 0; peer < world; ++peer) {
    if (receive_buffers[peer] == nullptr || !aligned16(receive_buffers[peer])) return -1;
    receive.base[peer] = receive_buffers[peer];
  }
  if (count == 0) return 0;
  return mircuda_b200::launch_after_dependency(moe_dispatch_rows_kernel, dim3(grid_for(count, kThreads / 32)), dim3(kThreads),
                                 0, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(source),
                                 source_index, sorted_expert, position, base_for_me, receive, remote_row, count,
                                 local_experts, columns / 8u, capacity_rows);
}

extern "C" int mircuda_b200_moe_collect_rows_bf16(
    void* const* result_buffers, uint32_t world, const int* slot, const int* sorted_expert,
    const int* remote_row, const float* weights, void* output, uint32_t tokens, uint32_t top_k,
    uint32_t local_experts, uint32_t columns, void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (result_buffers == nullptr || slot == nullptr || sorted_expert == nullptr ||
      remote_row == nullptr || weights == nullptr || output == nullptr || world == 0 || world > 8 ||
      top_k == 0 || top_k > 32 || local_experts == 0 || columns == 0 || columns % 8 != 0 || !aligned16(output)) {
    return -1;
  }
  PeerBases results = {};
  for (uint32_t peer = 0; peer < world; ++peer) {
    if (result_buffers[peer] == nullptr || !aligned16(result_buffers[peer])) return -1;
    results.base[peer] = result_buffers[peer];
  }
  if (tokens == 0) return 0;
  // Warps per token: enough for about 4096 warps in all, each with at least 32 pieces.
  const uint32_t pieces = columns / 8u;
  uint32_t parts = 1u;
  while (parts < 8u && tokens * parts < 4096u && pieces / (parts * 2u) >= 32u) parts *= 2u;
  const int grid = grid_for(static_cast<size_t>(tokens) * parts, kThreads / 32);
  auto cuda_stream = static_cast<cudaStream_t>(stream);
  return mircuda_b200::launch_after_dependency(top_k <= 8 ? moe_collect_rows_kernel<8> : moe_collect_rows_kernel<32>,
                                 dim3(grid), dim3(kThreads), 0, cuda_stream, results, slot, sorted_expert,
                                 remote_row, weights, static_cast<uint4*>(output), tokens, top_k, local_experts,
                                 pieces, parts);
}

extern "C" int mircuda_b200_moe_scale_atoms(const void* row_scales, void* atoms, uint32_t rows,
                                            const unsigned int* row_bound, uint32_t columns,
                                            void* stream) {
  using namespace mircuda_b200::moe_rows;
  if (row_scales == nullptr || atoms == nullptr || rows == 0 || columns == 0 || columns % 16 != 0 ||
      !aligned16(row_scales) || (reinterpret_cast<uintptr_t>(atoms) & 3u) != 0u) {
    return -1;
  }
  const size_t total = static_cast<size_t>(rows) * (columns / 16u);
  return mircuda_b200::launch_after_dependency(moe_scale_atoms_kernel, dim3(grid_for(total, kThreads)), dim3(kThreads), 0,
                                 static_cast<cudaStream_t>(stream), static_cast<const uint4*>(row_scales),
                                 static_cast<uint8_t*>(atoms), rows, row_bound, columns);
}
