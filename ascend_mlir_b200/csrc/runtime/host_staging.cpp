#include "runtime/host_staging.h"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstring>
#include <string>

namespace afir {

// ---- ParallelCopier ------------------------------------------------------------------------------------------------
ParallelCopier::ParallelCopier(int threads) {
  for (int i = 1; i < threads; ++i) workers_.emplace_back([this, i] { workerLoop(i); });
}

ParallelCopier::~ParallelCopier() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    stop_ = true;
  }
  wake_.notify_all();
  for (std::thread &t : workers_) t.join();
}

void ParallelCopier::workerLoop(int index) {
  uint64_t seen = 0;
  while (true) {
    char *dst;
    const char *src;
    size_t bytes, piece;
    {
      std::unique_lock<std::mutex> lock(mu_);
      wake_.wait(lock, [&] { return stop_ || generation_ != seen; });
      if (stop_) return;
      seen = generation_;
      dst = dst_; src = src_; bytes = bytes_; piece = piece_;
    }
    const size_t begin = std::min(bytes, piece * static_cast<size_t>(index));
    const size_t end = std::min(bytes, begin + piece);
    if (end > begin) std::memcpy(dst + begin, src + begin, end - begin);
    {
      std::lock_guard<std::mutex> lock(mu_);
      if (--pending_ == 0) done_.notify_one();
    }
  }
}

void ParallelCopier::copy(void *dst, const void *src, size_t bytes) {
  const size_t shares = workers_.size() + 1;
  if (bytes < (1u << 20) || shares == 1) {  // not worth waking anybody
    std::memcpy(dst, src, bytes);
    return;
  }
  const size_t piece = ((bytes + shares - 1) / shares + 4095) & ~static_cast<size_t>(4095);
  {
    std::lock_guard<std::mutex> lock(mu_);
    dst_ = static_cast<char *>(dst);
    src_ = static_cast<const char *>(src);
    bytes_ = bytes;
    piece_ = piece;
    pending_ = static_cast<int>(workers_.size());
    ++generation_;
  }
  wake_.notify_all();
  std::memcpy(dst, src, std::min(bytes, piece));  // share 0
  std::unique_lock<std::mutex> lock(mu_);
  done_.wait(lock, [&] { return pending_ == 0; });
}

// ---- HostStager ------------------------------------------------------------------------------------------------------
namespace {
Status cudaFail(cudaError_t e, const char *what) { return Status::error(std::string(what) + ": " + cudaGetErrorString(e)); }
} // namespace

HostStager::~HostStager() {
  for (Slot *set : {in_, out_})
    for (int i = 0; i < 2; ++i) {
      if (set[i].event) cudaEventDestroy(static_cast<cudaEvent_t>(set[i].event));
      if (set[i].pinned) cudaFreeHost(set[i].pinned);
    }
  delete copier_;
}

bool HostStager::isPageable(const void *p) {
  if (!p) return false;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();  // older drivers report unregistered host memory as an error: clear it
    return true;
  }
  return attr.type == cudaMemoryTypeUnregistered;
}

Status HostStager::prepare() {
  if (ready_) return Status::success();
  for (Slot *set : {in_, out_})
    for (int i = 0; i < 2; ++i) {
      cudaError_t e = cudaHostAlloc(&set[i].pinned, kSlotBytes, cudaHostAllocDefault);
      if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] pinned staging allocation failed");
      cudaEvent_t ev;
      e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
      if (e != cudaSuccess) return cudaFail(e, "[cuda:device] cudaEventCreate");
      set[i].event = ev;
    }
  const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  copier_ = new ParallelCopier(static_cast<int>(std::min(8u, std::max(1u, hw / 2))));
  ready_ = true;
  return Status::success();
}

Status HostStager::copyIn(void *device, const void *host, size_t bytes, cudaStream_t stream) {
  size_t off = 0;
  while (off < bytes) {
    const size_t n = std::min(kSlotBytes, bytes - off);
    Slot &slot = in_[inTurn_++ & 1u];
    if (slot.busy) {  // the DMA that last read this slot must be over before it is overwritten
      cudaError_t e = cudaEventSynchronize(static_cast<cudaEvent_t>(slot.event));
      if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] host-to-device copy failed");
      slot.busy = false;
    }
    copier_->copy(slot.pinned, static_cast<const char *>(host) + off, n);
    cudaError_t e = cudaMemcpyAsync(static_cast<char *>(device) + off, slot.pinned, n, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(static_cast<cudaEvent_t>(slot.event), stream);
    if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] host-to-device copy failed");
    slot.busy = true;
    off += n;
  }
  return Status::success();
}

Status HostStager::drain(Slot &slot) {
  if (!slot.busy) return Status::success();
  cudaError_t e = cudaEventSynchronize(static_cast<cudaEvent_t>(slot.event));
  slot.busy = false;
  if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] device-to-host copy failed");
  copier_->copy(slot.hostDst, slot.pinned, slot.bytes);
  return Status::success();
}

Status HostStager::copyOut(void *host, const void *device, size_t bytes, cudaStream_t stream) {
  size_t off = 0;
  while (off < bytes) {
    const size_t n = std::min(kSlotBytes, bytes - off);
    Slot &slot = out_[outTurn_++ & 1u];
    if (Status s = drain(slot); !s) return s;  // what the slot still holds goes to its destination first
    cudaError_t e = cudaMemcpyAsync(slot.pinned, static_cast<const char *>(device) + off, n, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaEventRecord(static_cast<cudaEvent_t>(slot.event), stream);
    if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] device-to-host copy failed");
    slot.busy = true;
    slot.hostDst = static_cast<char *>(host) + off;
    slot.bytes = n;
    off += n;
  }
  return Status::success();
}

Status HostStager::finishOut() {
  // oldest first
  for (unsigned k = 0; k < 2; ++k)
    if (Status s = drain(out_[(outTurn_ + k) & 1u]); !s) return s;
  return Status::success();
}

} // namespace afir
