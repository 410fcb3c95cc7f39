// All-gather of column blocks with the copy engines (multi-GPU linears whose weights are sharded
// along N). Every rank holds a full-width [rows, pitch] output in peer-mapped memory and has just
// written its own column block of it; `send` copies that block into the same place of every
// peer's buffer with one strided device-to-device copy per peer, each on a stream of its own so
// that the copies to different peers run on different engines. The copies wait for the compute
// stream at the point of the call and the compute stream goes on at once: the transfer of one
// layer overlaps the kernels of the next and takes no store slots of the SMs. `join` makes the
// compute stream wait for every copy issued so far; the caller then synchronises the ranks
// (a stream-ordered barrier) before anything reads the gathered outputs or overwrites a block
// that may still be in flight. The same calls carry the other layout of an all-gather, rank-major
// blocks (rank r's [rows, local columns] matrix at block r of every buffer): a block is contiguous
// and goes as a 1-D copy, which the engines move faster than narrow row segments. One plain
// asynchronous copy per peer and call; nothing here waits on the host.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <new>

namespace mircuda_b200 {
namespace column_gather {

constexpr uint32_t kMaxWorld = 8;

struct Gather {
  uint32_t world, rank;
  int device;
  cudaStream_t streams[kMaxWorld];   // one per peer (the own slot stays null)
  cudaEvent_t ready;                 // recorded on the compute stream at every send
  cudaEvent_t done[kMaxWorld];       // recorded on a peer's stream at every join
  bool pending;
};

void release(Gather* gather) {
  if (gather == nullptr) return;
  for (uint32_t peer = 0; peer < kMaxWorld; ++peer) {
    if (gather->streams[peer] != nullptr) cudaStreamDestroy(gather->streams[peer]);
    if (gather->done[peer] != nullptr) cudaEventDestroy(gather->done[peer]);
  }
  if (gather->ready != nullptr) cudaEventDestroy(gather->ready);
  delete gather;
}

}  // namespace column_gather
}  // namespace mircuda_b200

using mircuda_b200::column_gather::Gather;
using mircuda_b200::column_gather::kMaxWorld;

extern "C" int mircuda_b200_column_gather_create(uint32_t world, uint32_t rank, void** output) {
  if (world < 2 || world > kMaxWorld || rank >= world || output == nullptr) return -1;
  auto* gather = new (std::nothrow) Gather{};
  if (gather == nullptr) return -2;
  gather->world = world;
  gather->rank = rank;
  int status = static_cast<int>(cudaGetDevice(&gather->device));
  if (status == 0) status = static_cast<int>(cudaEventCreateWithFlags(&gather->ready, cudaEventDisableTiming));
  for (uint32_t peer = 0; peer < world && status == 0; ++peer) {
    if (peer == rank) continue;
    status = static_cast<int>(cudaStreamCreateWithFlags(&gather->streams[peer], cudaStreamNonBlocking));
    if (status == 0) {
      status = static_cast<int>(cudaEventCreateWithFlags(&gather->done[peer], cudaEventDisableTiming));
    }
  }
  if (status != 0) {
    mircuda_b200::column_gather::release(gather);
    return status;
  }
  *output = gather;
  return 0;
}

// buffers[p]: rank p's output buffer as mapped into this process (buffers[rank] is the own one);
// the block is `rows` rows of `width_bytes`, `pitch_bytes` apart, the first starting
// `offset_bytes` into the buffer: a column block of a full-width matrix, or (one row, or rows
// that follow one another) a contiguous piece, which is sent with a 1-D copy.
extern "C" int mircuda_b200_column_gather_send(void* raw, void* const* buffers, uint64_t pitch_bytes,
                                               uint64_t offset_bytes, uint64_t width_bytes,
                                               uint64_t rows, void* stream) {
  auto* gather = static_cast<Gather*>(raw);
  if (gather == nullptr || buffers == nullptr || stream == nullptr || pitch_bytes == 0 || width_bytes == 0 ||
      rows == 0 || width_bytes > pitch_bytes) {
    return -1;
  }
  const bool contiguous = rows == 1 || width_bytes == pitch_bytes;
  for (uint32_t peer = 0; peer < gather->world; ++peer) {
    if (buffers[peer] == nullptr) return -1;
  }
  int status = static_cast<int>(cudaEventRecord(gather->ready, static_cast<cudaStream_t>(stream)));
  const uint8_t* source = static_cast<const uint8_t*>(buffers[gather->rank]) + offset_bytes;
  // Peers in the order rank + 1, rank + 2, ...: at any moment the ranks send to different peers.
  for (uint32_t step = 1; step < gather->world && status == 0; ++step) {
    const uint32_t peer = (gather->rank + step) % gather->world;
    status = static_cast<int>(cudaStreamWaitEvent(gather->streams[peer], gather->ready, 0));
    if (status != 0) break;
    uint8_t* destination = static_cast<uint8_t*>(buffers[peer]) + offset_bytes;
    status = contiguous
                 ? static_cast<int>(cudaMemcpyAsync(destination, source, width_bytes * rows, cudaMemcpyDefault,
                                                    gather->streams[peer]))
                 : static_cast<int>(cudaMemcpy2DAsync(destination, pitch_bytes, source, pitch_bytes, width_bytes,
                                                      rows, cudaMemcpyDefault, gather->streams[peer]));
  }
  gather->pending = true;
  return status;
}

extern "C" int mircuda_b200_column_gather_join(void* raw, void* stream) {
  auto* gather = static_cast<Gather*>(raw);
  if (gather == nullptr || stream == nullptr) return -1;
  if (!gather->pending) return 0;
  int status = 0;
  for (uint32_t peer = 0; peer < gather->world && status == 0; ++peer) {
    if (peer == gather->rank) continue;
    status = static_cast<int>(cudaEventRecord(gather->done[peer], gather->streams[peer]));
    if (status == 0) {
      status = static_cast<int>(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), gather->done[peer], 0));
    }
  }
  gather->pending = false;
  return status;
}

// The caller has synchronised the streams that `send` was given.
extern "C" void mircuda_b200_column_gather_destroy(void* raw) {
  auto* gather = static_cast<Gather*>(raw);
  if (gather == nullptr) return;
  for (uint32_t peer = 0; peer < kMaxWorld; ++peer) {
    if (gather->streams[peer] != nullptr) cudaStreamSynchronize(gather->streams[peer]);
  }
  mircuda_b200::column_gather::release(gather);
}
