// The stateless Marlin entry points have no plan to carry a status word for the bounded waits of
// their streaming kernels, so the process keeps one pinned word: a launch whose wait ran out sets
// it and every later call returns -3. It is allocated by the first call that is not being
// captured into a graph; until it exists (a first call under capture) kernels run without a
// place to report to.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>
#include <mutex>

namespace mircuda_b200 {

// Returns the word (or null while it cannot be allocated); `*failed` says whether an earlier
// launch has set it.
inline uint32_t* marlin_status_word(cudaStream_t stream, bool* failed) {
  static std::mutex guard;
  static uint32_t* word = nullptr;
  {
    std::lock_guard<std::mutex> hold(guard);
    if (word == nullptr) {
      cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(stream, &capture) == cudaSuccess && capture == cudaStreamCaptureStatusNone) {
        void* memory = nullptr;
        if (cudaHostAlloc(&memory, sizeof(uint32_t), cudaHostAllocPortable) == cudaSuccess) {
          word = static_cast<uint32_t*>(memory);
          *word = 0u;
        }
      }
    }
  }
  *failed = word != nullptr && *reinterpret_cast<volatile uint32_t*>(word) != 0u;
  return word;
}

}  // namespace mircuda_b200
