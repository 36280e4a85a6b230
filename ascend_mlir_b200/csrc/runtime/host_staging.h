// Staging of PAGEABLE host buffers through pinned memory.  The reference-side caller of afirt_executor_run hands
// over ordinary host arrays (numpy); a cudaMemcpyAsync from pageable memory is staged by the driver in one thread
// and does not overlap with anything, which made the end-to-end path six times slower than with pinned buffers.
// Here the executor owns two pinned slots per direction and a few worker threads: a piece of the caller's buffer
// is copied into a free slot by all workers at once while the previous slot's DMA and the kernels are still running,
// and results come back the same way.  One cudaMemcpyAsync per piece; nothing is batched.
#pragma once

#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "common/status.h"

typedef struct CUstream_st *cudaStream_t;

namespace afir {

// A few persistent threads that copy one byte range in parallel (the calling thread takes a share too).
class ParallelCopier {
public:
  explicit ParallelCopier(int threads);
  ~ParallelCopier();
  ParallelCopier(const ParallelCopier &) = delete;
  ParallelCopier &operator=(const ParallelCopier &) = delete;
  void copy(void *dst, const void *src, size_t bytes);
  int threads() const { return static_cast<int>(workers_.size()) + 1; }

private:
  void workerLoop(int index);
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable wake_, done_;
  uint64_t generation_ = 0;
  int pending_ = 0;
  bool stop_ = false;
  char *dst_ = nullptr;
  const char *src_ = nullptr;
  size_t bytes_ = 0, piece_ = 0;
};

class HostStager {
public:
  static constexpr size_t kSlotBytes = 16u << 20;
  HostStager() = default;
  ~HostStager();
  HostStager(const HostStager &) = delete;
  HostStager &operator=(const HostStager &) = delete;

  // True when `p` is ordinary pageable host memory (not pinned, not registered, not managed).
  static bool isPageable(const void *p);

  // Allocates the pinned slots and events and starts the workers on first use.
  Status prepare();
  // Host -> device through the slots; returns once the last piece has been handed to the copy engine on `stream`
  // (the caller's buffer may be reused then; the device copy completes in stream order).
  Status copyIn(void *device, const void *host, size_t bytes, cudaStream_t stream);
  // Device -> host through the slots, on `stream` (which the caller has already ordered after the producing
  // kernel).  Pieces land in the caller's buffer when their slot is needed again or at finishOut().
  Status copyOut(void *host, const void *device, size_t bytes, cudaStream_t stream);
  // Waits for every piece still in a slot and copies it to its destination.
  Status finishOut();

private:
  struct Slot {
    void *pinned = nullptr;
    void *event = nullptr;   // recorded after the DMA that uses the slot
    bool busy = false;       // an event has been recorded and not yet waited for
    void *hostDst = nullptr; // out slots: where the piece goes
    size_t bytes = 0;
  };
  Status drain(Slot &slot);
  Slot in_[2], out_[2];
  unsigned inTurn_ = 0, outTurn_ = 0;
  bool ready_ = false;
  ParallelCopier *copier_ = nullptr;
};

} // namespace afir
