// CUDA execution runner: the B200 counterpart of the reference's NativeExecutionRunner
// (lib/Runtime/Execution/NativeExecutionRunner.cpp:126-154,372-528): per call it stages the
// inputs on the device, launches the kernel named by the binary, waits, and copies the outputs
// back.  Device buffers are pooled per executor instead of being allocated and freed per call.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "runtime/descriptor.h"
#include "runtime/host_staging.h"
#include "runtime/launcher.h"

namespace afir {

constexpr uint32_t kMagicVec = 0x41415246u;   // vector / mixed kernels
constexpr uint32_t kMagicCube = 0x41494343u;  // cube (matmul-only) kernels

struct RunRequest {
  const uint8_t *binary = nullptr;
  size_t binaryLen = 0;
  std::string functionName;
  int numInputs = 0;
  const void *const *inputPtrs = nullptr;
  const size_t *inputBytes = nullptr;
  int numOutputs = 0;
  void *const *outputPtrs = nullptr;
  const size_t *outputBytes = nullptr;
  const uint8_t *tiling = nullptr;
  size_t tilingLen = 0;
  int blockDim = 0;
  uint32_t magic = kMagicVec;
};

class CudaExecutor {
public:
  CudaExecutor() = default;
  ~CudaExecutor();
  CudaExecutor(const CudaExecutor &) = delete;
  CudaExecutor &operator=(const CudaExecutor &) = delete;

  Status initialize(int deviceId);
  bool initialized() const { return initialized_; }
  int device() const { return device_; }

  // Host-pointer path: H2D, launch, D2H, synchronise, status checks.
  Status runHost(const RunRequest &req);
  // Device-pointer path: validates and enqueues the launch on `stream` and returns.
  // exchange: not null for a row-reduction group whose reduced axis is sharded over GPUs (the kernel then
  // exchanges its partial sums through that mailbox record)
  // tableShards / rowsPerShard: not empty for a row-gather group whose table is given as row shards (possibly
  // other GPUs' memory, peer-mapped) instead of its one argument
  Status launchDevice(const RunRequest &req, void *workspace, size_t workspaceBytes, void *stream,
                      const kernels::RowReduceExchange *exchange = nullptr,
                      const std::vector<const void *> &tableShards = {}, int64_t rowsPerShard = 0);
  // Waits for `stream` (null = the executor's own) and surfaces device-side status words.
  Status synchronize(void *stream);

  // Re-launches the kernel of `req` on the device buffers the last runHost of the same request left
  // resident and returns the median kernel time over `repeats` launches (CUDA events on the executor stream).
  Status profileResident(const RunRequest &req, int repeats, double &medianMicroseconds);

  // True when the last launch ran the group's generated kernel (compiled from its own source), false when it ran
  // a prebuilt kernel of the library.
  bool lastLaunchGenerated() const { return lastLaunchGenerated_; }
  int lastLaunchCount() const { return lastLaunchCount_; }
  uint64_t totalLaunchCount() const { return totalLaunchCount_; }

private:
  struct Slot { void *ptr = nullptr; size_t capacity = 0; };
  // One kernel binary this executor has met: its descriptor and, once a launch wanted it, its generated kernel
  // loaded on the executor's device (the reference's runner caches registered binaries the same way,
  // lib/Runtime/Execution/NativeExecutionRunner.cpp:332).
  struct CachedKernel {
    std::shared_ptr<const LaunchDescriptor> desc;
    std::vector<uint8_t> cubin;   // from the container; empty = compile on first use
    bool generatedTried = false;
    bool generatedUsable = false;
    std::string generatedNote;    // why not, when unusable
    GeneratedBinding binding;
  };
  Status validate(const RunRequest &req, CachedKernel *&kernel, std::map<std::string, int64_t> &tiling);
  // Loads (compiling first when the container brought no device binary) the kernel's generated code.
  bool prepareGenerated(CachedKernel &kernel);
  // Runs the descriptor on its generated kernel when the policy (AFIR_CUDA_CODEGEN = auto | always | never) and
  // the launch allow it, on the library's prebuilt kernels otherwise.
  Status dispatch(CachedKernel &kernel, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args, LaunchInfo &info);
  Status slotFor(size_t index, size_t bytes, void **out);
  Status ensureStream();
  Status ownWorkspace(size_t bytes);
  // Host path cut into leading-axis chunks: H2D of chunk i+1, the kernel on chunk i and D2H of chunk i-1 overlap.
  Status runHostPipelined(const RunRequest &req, CachedKernel &kernel, const std::map<std::string, int64_t> &tiling,
                          LaunchArgs &args, const RowPipelinePlan &plan, int64_t chunkRows);
  Status ensureCopyStreams(size_t events);

  bool initialized_ = false;
  int device_ = 0;
  void *stream_ = nullptr;
  void *copyIn_ = nullptr;
  void *copyOut_ = nullptr;
  std::vector<void *> events_;
  // Pageable host buffers (what a numpy caller hands over) go through pinned slots filled by several threads;
  // AFIR_CUDA_NO_STAGING=1 leaves them to the driver's own single-threaded staging.
  std::unique_ptr<HostStager> stager_;
  // Copies between the caller's buffers and the device, through the stager when the host side is pageable and large.
  Status copyToDevice(void *device, const void *host, size_t bytes, void *stream);
  Status copyToHost(void *host, const void *device, size_t bytes, void *stream);
  std::vector<Slot> slots_;
  Slot workspace_;
  std::unordered_map<uint64_t, CachedKernel> cache_;
  int lastLaunchCount_ = 0;
  bool lastLaunchGenerated_ = false;
  uint64_t totalLaunchCount_ = 0;
  bool statusPending_ = false;
  void *statusWorkspace_ = nullptr;
  // Debug guard bands (AFIR_CUDA_CANARY=1): every host-path buffer gets `guard` bytes of a known pattern before and
  // after it; the bands of the outputs are checked after the run, so a kernel that writes outside its output
  // shows up as an error instead of silent corruption of a neighbouring allocation.
  struct GuardCheck { int output; const unsigned char *before; const unsigned char *after; };
  std::vector<GuardCheck> guardChecks_;
  size_t guardBytes_ = 0;
  Status verifyGuards();
  bool matmulPending_ = false;
  bool transposePending_ = false;  // a transpose-capable launch ran without a status block: the library's own word is checked
  bool reducePending_ = false;
};

} // namespace afir
