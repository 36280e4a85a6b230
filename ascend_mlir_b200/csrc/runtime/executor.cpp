#include "runtime/executor.h"

#include <cuda_runtime_api.h>

#include "codegen/nvrtc_compile.h"

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace afir {
namespace {

Status cudaFail(cudaError_t e, const char *what) {
  return Status::error(std::string(what) + ": " + cudaGetErrorString(e));
}

uint64_t fnv1a(const uint8_t *p, size_t n) {
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
  return h ^ (static_cast<uint64_t>(n) << 1);
}

} // namespace

CudaExecutor::~CudaExecutor() {
  if (!initialized_) return;
  if (cudaSetDevice(device_) != cudaSuccess) return;
  for (auto &s : slots_)
    if (s.ptr) cudaFree(s.ptr);
  if (workspace_.ptr) cudaFree(workspace_.ptr);
  if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
  if (copyIn_) cudaStreamDestroy(static_cast<cudaStream_t>(copyIn_));
  if (copyOut_) cudaStreamDestroy(static_cast<cudaStream_t>(copyOut_));
  for (void *e : events_) cudaEventDestroy(static_cast<cudaEvent_t>(e));
}

Status CudaExecutor::initialize(int deviceId) {
  if (deviceId < 0) return Status::error("device id must be non-negative");
  device_ = deviceId;
  initialized_ = true;  // the device itself is first touched by the first run (the reference defers too)
  return Status::success();
}

Status CudaExecutor::ensureStream() {
  cudaError_t e = cudaSetDevice(device_);
  if (e != cudaSuccess) return cudaFail(e, "cudaSetDevice");
  if (!stream_) {
    cudaStream_t s;
    e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    if (e != cudaSuccess) return cudaFail(e, "cudaStreamCreate");
    stream_ = s;
  }
  return Status::success();
}

Status CudaExecutor::slotFor(size_t index, size_t bytes, void **out) {
  if (slots_.size() <= index) slots_.resize(index + 1);
  Slot &s = slots_[index];
  const size_t need = bytes ? bytes : 16;
  if (s.capacity < need) {
    if (s.ptr) cudaFree(s.ptr);
    s.ptr = nullptr;
    s.capacity = 0;
    cudaError_t e = cudaMalloc(&s.ptr, need);
    if (e != cudaSuccess) return cudaFail(e, "device allocation failed");
    s.capacity = need;
  }
  *out = s.ptr;
  return Status::success();
}

// Launch-time failures are kernel_launch errors unless the launcher already named a more precise stage
// (a tensor whose byte count contradicts the tiling dims is a bindings error).
static Status launchStage(const Status &s) {
  if (s.ok() || (!s.message().empty() && s.message()[0] == '[')) return s;
  return s.withStage("cuda:kernel_launch");
}

static size_t guardBytesFromEnv() {
  const char *v = std::getenv("AFIR_CUDA_CANARY");
  if (!v || !*v || std::string(v) == "0") return 0;
  return 4096;  // a multiple of 512, so buffers keep the alignment cudaMalloc gave them
}
static constexpr unsigned char kGuardPattern = 0xA5;

Status CudaExecutor::verifyGuards() {
  if (guardChecks_.empty()) return Status::success();
  std::vector<unsigned char> host(2 * guardBytes_);
  Status result = Status::success();
  for (const GuardCheck &g : guardChecks_) {
    cudaError_t e = cudaMemcpy(host.data(), g.before, guardBytes_, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(host.data() + guardBytes_, g.after, guardBytes_, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { result = cudaFail(e, "[cuda:memory] guard band read failed"); break; }
    for (size_t i = 0; i < host.size(); ++i) {
      if (host[i] == kGuardPattern) continue;
      const bool before = i < guardBytes_;
      const long long off = before ? static_cast<long long>(i) - static_cast<long long>(guardBytes_) : static_cast<long long>(i - guardBytes_);
      result = Status::error("[cuda:kernel_launch] output " + std::to_string(g.output) + ": the kernel wrote " +
                             (before ? "before the start" : "past the end") + " of the buffer (first bad byte at offset " +
                             std::to_string(off) + (before ? " from the start)" : " from the end)"));
      break;
    }
    if (!result) break;
  }
  guardChecks_.clear();
  return result;
}

Status CudaExecutor::ownWorkspace(size_t bytes) {
  if (workspace_.capacity >= bytes) return Status::success();
  if (workspace_.ptr) cudaFree(workspace_.ptr);
  workspace_ = Slot();
  cudaError_t e = cudaMalloc(&workspace_.ptr, bytes);
  if (e != cudaSuccess) return cudaFail(e, "workspace allocation failed");
  workspace_.capacity = bytes;
  return Status::success();
}

// ASCEND_RUNTIME_TRACE_LAUNCH / AFIR_CUDA_TRACE_LAUNCH set to anything but 0/false/off/no: every launch prints
// its arguments, their alignment and the tiling words to stderr, in the line format of the reference's launch
// trace (lib/Runtime/Execution/LaunchTrace.cpp:40-103) with "cuda-launch" as the tag.
static bool launchTraceEnabled() {
  for (const char *name : {"ASCEND_RUNTIME_TRACE_LAUNCH", "AFIR_CUDA_TRACE_LAUNCH"}) {
    const char *raw = std::getenv(name);
    if (!raw || !*raw) continue;
    std::string v(raw);
    for (char &c : v) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    if (v != "0" && v != "false" && v != "off" && v != "no") return true;
  }
  return false;
}

// First bytes of a buffer as hex, the reference's printNativeLaunchBufferSample line
// (lib/Runtime/Execution/LaunchTrace.cpp:93-101; 64 bytes, NativeExecutionRunner.cpp:63).
static constexpr size_t kLaunchTraceSampleBytes = 64;
static void printBufferSample(const std::string &label, const unsigned char *bytes, size_t sampleBytes, size_t totalBytes) {
  std::string hex;
  static const char digits[] = "0123456789abcdef";
  for (size_t i = 0; i < sampleBytes; ++i) { hex += digits[bytes[i] >> 4]; hex += digits[bytes[i] & 15]; }
  std::fprintf(stderr, "[cuda-launch] %s bytes=%zu sample_bytes=%zu sample_hex=%s\n", label.c_str(), totalBytes, sampleBytes, hex.c_str());
}

static void printLaunchTrace(const RunRequest &req, const LaunchDescriptor &desc, const LaunchArgs &args, int device, const char *path) {
  auto ptr = [](const void *p) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "%p align512=%s", p, (reinterpret_cast<uintptr_t>(p) & 511u) == 0 ? "yes" : "no");
    return std::string(buf);
  };
  std::fprintf(stderr, "[cuda-launch] kernel=%s class=%d path=%s magic=0x%08x device_id=%d block_dim=%d args_count=%d\n",
               desc.kernel.c_str(), static_cast<int>(desc.kernelClass), path, req.magic, device, req.blockDim,
               req.numInputs + req.numOutputs + 2);
  std::fprintf(stderr, "[cuda-launch] inputs=%d outputs=%d workspace_size=%zu tiling_bytes=%zu tiling_words=%zu\n", req.numInputs,
               req.numOutputs, args.workspaceBytes, req.tilingLen, (req.tilingLen + 7) / 8);
  for (int i = 0; i < req.numInputs; ++i)
    std::fprintf(stderr, "[cuda-launch] input[%d] bytes=%zu ptr=%s\n", i, args.argBytes[i], ptr(args.argPtrs[i]).c_str());
  for (int i = 0; i < req.numOutputs; ++i)
    std::fprintf(stderr, "[cuda-launch] output[%d] bytes=%zu ptr=%s\n", i, args.argBytes[req.numInputs + i],
                 ptr(args.argPtrs[req.numInputs + i]).c_str());
  std::fprintf(stderr, "[cuda-launch] workspace bytes=%zu ptr=%s\n", args.workspaceBytes, ptr(args.workspace).c_str());
  const size_t words = std::min<size_t>((req.tilingLen + 7) / 8, 32);
  for (size_t w = 0; w < words; ++w) {
    uint64_t v = 0;
    std::memcpy(&v, req.tiling + w * 8, std::min<size_t>(8, req.tilingLen - w * 8));
    const char *name = w < desc.tiling.size() ? desc.tiling[w].name.c_str() : "";
    std::fprintf(stderr, "[cuda-launch] tiling.word[%zu]=%llu %s\n", w, static_cast<unsigned long long>(v), name);
  }
}

Status CudaExecutor::validate(const RunRequest &req, CachedKernel *&kernel, std::map<std::string, int64_t> &tiling) {
  std::shared_ptr<const LaunchDescriptor> desc;
  if (!initialized_) return Status::error("executor has not been initialized");
  if (!req.binary || req.binaryLen == 0) return Status::error("binary data is required");
  if (req.functionName.empty()) return Status::error("function name is required");
  if (req.numInputs < 0 || req.numOutputs <= 0) return Status::error("invalid input/output binding counts");
  if ((req.numInputs > 0 && (!req.inputPtrs || !req.inputBytes)) || !req.outputPtrs || !req.outputBytes)
    return Status::error("input/output pointer arrays are required");
  if (req.magic != kMagicVec && req.magic != kMagicCube) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "unsupported kernel magic: 0x%08x", req.magic);
    return Status::error(buf);
  }
  const uint64_t key = fnv1a(req.binary, req.binaryLen);
  auto it = cache_.find(key);
  if (it == cache_.end()) {
    auto d = std::make_shared<LaunchDescriptor>();
    if (Status s = parseDescriptorBinary(req.binary, req.binaryLen, *d); !s) return s.withStage("cuda:artifact");
    CachedKernel fresh;
    fresh.desc = std::move(d);
    const ContainerCode code = containerCode(req.binary, req.binaryLen);
    if (code.cubinLen) fresh.cubin.assign(code.cubin, code.cubin + code.cubinLen);
    it = cache_.emplace(key, std::move(fresh)).first;
  }
  kernel = &it->second;
  desc = kernel->desc;
  if (desc->kernel != req.functionName)
    return Status::error("[cuda:artifact] kernel binary defines '" + desc->kernel + "', not '" + req.functionName + "'");
  if (req.numInputs != desc->numInputs || req.numOutputs != desc->numOutputs)
    return Status::error("[cuda:bindings] kernel '" + desc->kernel + "' takes " + std::to_string(desc->numInputs) +
                         " inputs and " + std::to_string(desc->numOutputs) + " outputs, got " +
                         std::to_string(req.numInputs) + " and " + std::to_string(req.numOutputs));
  for (int i = 0; i < req.numInputs; ++i)
    if (!req.inputPtrs[i] && req.inputBytes[i]) return Status::error("[cuda:bindings] input " + std::to_string(i) + " is null");
  for (int i = 0; i < req.numOutputs; ++i)
    if (!req.outputPtrs[i] && req.outputBytes[i]) return Status::error("[cuda:bindings] output " + std::to_string(i) + " is null");
  if (Status s = unpackTiling(*desc, req.tiling, req.tilingLen, tiling); !s) return s.withStage("cuda:bindings");
  return Status::success();
}

// Below this size the driver's own staging of a pageable buffer is not worth replacing.
static constexpr size_t kStagingMinBytes = 1u << 20;
static bool stagingEnabled() {
  const char *v = std::getenv("AFIR_CUDA_NO_STAGING");
  return !(v && *v && std::string(v) != "0");
}

Status CudaExecutor::copyToDevice(void *device, const void *host, size_t bytes, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bytes >= kStagingMinBytes && stagingEnabled() && HostStager::isPageable(host)) {
    if (!stager_) stager_.reset(new HostStager());
    if (Status st = stager_->prepare(); !st) return st;
    return stager_->copyIn(device, host, bytes, s);
  }
  const cudaError_t e = cudaMemcpyAsync(device, host, bytes, cudaMemcpyHostToDevice, s);
  return e == cudaSuccess ? Status::success() : cudaFail(e, "[cuda:memory] host-to-device copy failed");
}

Status CudaExecutor::copyToHost(void *host, const void *device, size_t bytes, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bytes >= kStagingMinBytes && stagingEnabled() && HostStager::isPageable(host)) {
    if (!stager_) stager_.reset(new HostStager());
    if (Status st = stager_->prepare(); !st) return st;
    return stager_->copyOut(host, device, bytes, s);
  }
  const cudaError_t e = cudaMemcpyAsync(host, device, bytes, cudaMemcpyDeviceToHost, s);
  return e == cudaSuccess ? Status::success() : cudaFail(e, "[cuda:memory] device-to-host copy failed");
}

// AFIR_CUDA_CODEGEN: "auto" (default) and "always" run elementwise / split / concat, row-reduction and row-gather
// groups on the kernel generated for them whenever one exists and the launch uses nothing the generated code leaves
// to the library (an exchange between GPUs, a sharded table, a tuning value of the library's own loops): measured
// at or above the library's straight-line kernels on every benchmark shape.  "never" keeps every launch on the
// library's prebuilt kernels.
static int codegenMode() {
  const char *v = std::getenv("AFIR_CUDA_CODEGEN");
  if (!v || !*v) return 1;
  const std::string s(v);
  if (s == "never" || s == "0" || s == "off") return 0;
  if (s == "always" || s == "2") return 2;
  return 1;
}

bool CudaExecutor::prepareGenerated(CachedKernel &kernel) {
  if (kernel.generatedTried) return kernel.generatedUsable;
  kernel.generatedTried = true;
  const LaunchDescriptor &d = *kernel.desc;
  const uint8_t *cubin = kernel.cubin.data();
  size_t cubinLen = kernel.cubin.size();
  std::shared_ptr<const std::vector<uint8_t>> compiled;
  if (cubinLen == 0) {
    // a descriptor that did not go through afirt_compiler_compile: generate and compile now
    const codegen::GeneratedKernel gen = codegen::generateKernelSource(d);
    if (!gen.supported) { kernel.generatedNote = gen.whyNot; return false; }
    if (Status s = codegen::compileToCubinCached(gen, compiled); !s) { kernel.generatedNote = s.message(); return false; }
    cubin = compiled->data();
    cubinLen = compiled->size();
  }
  if (Status s = DeviceModule::load(cubin, cubinLen, device_, kernel.binding.module); !s) { kernel.generatedNote = s.message(); return false; }
  if (Status s = kernel.binding.module->function(d.kernel, kernel.binding.mainFn); !s) { kernel.generatedNote = s.message(); return false; }
  if (d.kernelClass == KernelClass::RowReduce) {
    // optional entries: a module without them simply never takes that plan
    if (!kernel.binding.module->function(d.kernel + "__staged", kernel.binding.stagedFn)) kernel.binding.stagedFn = nullptr;
    if (!kernel.binding.module->function(d.kernel + "__finalize", kernel.binding.finalizeFn)) kernel.binding.finalizeFn = nullptr;
  }
  if (d.kernelClass == KernelClass::Gather &&
      !kernel.binding.module->function(d.kernel + "__one", kernel.binding.singleVectorFn))
    kernel.binding.singleVectorFn = nullptr;  // a module from before that entry existed: the main entry does everything
  void *marker = nullptr;  // present in modules whose kernels wait for their grid dependencies themselves
  kernel.binding.waitsForDependencies = static_cast<bool>(kernel.binding.module->function(codegen::kGridDependencyMarker, marker));
  kernel.binding.ctasOf256Threads = static_cast<bool>(kernel.binding.module->function(codegen::kRegisterBlockMarker, marker));
  kernel.generatedUsable = true;
  return true;
}

Status CudaExecutor::dispatch(CachedKernel &kernel, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args, LaunchInfo &info) {
  const LaunchDescriptor &d = *kernel.desc;
  const int mode = codegenMode();
  const bool classHasCode = d.kernelClass == KernelClass::Elementwise || d.kernelClass == KernelClass::RowReduce ||
                            d.kernelClass == KernelClass::Gather;
  if (mode != 0 && classHasCode && !(kernel.generatedTried && !kernel.generatedUsable) &&
      generatedLaunchApplies(d, tiling, args) &&
      prepareGenerated(kernel)) {
    Status s = launchGenerated(d, tiling, args, kernel.binding, info);
    // sizes the generated loop does not count (beyond 32 bits of elements) go to the library's kernels
    if (s || s.message().rfind("[generated:unsupported]", 0) != 0) return s;
  }
  return launchDescriptor(d, tiling, args, info);
}

Status CudaExecutor::runHost(const RunRequest &req) {
  CachedKernel *kernel = nullptr;
  std::map<std::string, int64_t> tiling;
  if (Status s = validate(req, kernel, tiling); !s) return s;
  const std::shared_ptr<const LaunchDescriptor> desc = kernel->desc;
  if (Status s = ensureStream(); !s) return s.withStage("cuda:device");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  LaunchArgs args;
  args.device = device_;
  args.stream = stream;
  args.blockDim = req.blockDim;
  const size_t numArgs = static_cast<size_t>(req.numInputs + req.numOutputs);
  args.argPtrs.resize(numArgs);
  args.argBytes.resize(numArgs);
  guardBytes_ = guardBytesFromEnv();
  guardChecks_.clear();
  const size_t guard = guardBytes_;
  for (int i = 0; i < req.numInputs; ++i) {
    args.argBytes[i] = req.inputBytes[i];
    void *base = nullptr;
    if (Status s = slotFor(i, req.inputBytes[i] + 2 * guard, &base); !s) return s.withStage("cuda:memory");
    args.argPtrs[i] = static_cast<char *>(base) + guard;
  }
  for (int i = 0; i < req.numOutputs; ++i) {
    const size_t k = static_cast<size_t>(req.numInputs + i);
    args.argBytes[k] = req.outputBytes[i];
    void *base = nullptr;
    if (Status s = slotFor(k, req.outputBytes[i] + 2 * guard, &base); !s) return s.withStage("cuda:memory");
    args.argPtrs[k] = static_cast<char *>(base) + guard;
    if (guard) {
      unsigned char *b = static_cast<unsigned char *>(base);
      unsigned char *after = b + guard + req.outputBytes[i];
      // bands are written on the compute stream, ahead of every kernel of this run
      cudaError_t ge = cudaMemsetAsync(b, kGuardPattern, guard, stream);
      if (ge == cudaSuccess) ge = cudaMemsetAsync(after, kGuardPattern, guard, stream);
      if (ge != cudaSuccess) return cudaFail(ge, "[cuda:memory] guard band fill failed");
      guardChecks_.push_back({i, b, after});
    }
  }
  size_t wsBytes = 0;
  if (Status s = requiredWorkspaceBytes(*desc, tiling, device_, wsBytes); !s) return s.withStage("cuda:bindings");
  if (Status s = ownWorkspace(wsBytes); !s) return s.withStage("cuda:memory");
  args.workspace = workspace_.ptr;
  args.workspaceBytes = workspace_.capacity;
  if (launchTraceEnabled()) printLaunchTrace(req, *desc, args, device_, "host");

  // Large runs whose work splits along the leading axis are pipelined: copies in, kernel and copies out
  // of successive row chunks overlap (PCIe is full duplex), instead of three serial phases.
  {
    RowPipelinePlan plan;
    if (Status s = planRowPipeline(*desc, tiling, args.argBytes, plan); !s) return s.withStage("cuda:bindings");
    size_t total = 0;
    for (size_t b : args.argBytes) total += b;
    // (not while tracing: the trace samples every buffer right after its copy, which wants the three plain phases)
    if (plan.possible && total >= (16u << 20) && plan.rows >= 2 && !std::getenv("AFIR_CUDA_NO_PIPELINE") && !launchTraceEnabled()) {
      const int64_t quantum = desc->kernelClass == KernelClass::Matmul ? 256 : (plan.rows >= 64 ? 8 : 1);
      // Chunks of about 16 MiB of sliced bytes, 4 to 12 of them: the copy-in stream never idles, so the time
      // not hidden is one chunk's kernel and copy-out at the end; smaller chunks shorten that tail until the
      // per-copy launch cost (a few microseconds each) starts to show (measured: flat from 8 to 24 chunks
      // on 192 MiB, slower again at 32).
      size_t sliced = 0;
      for (size_t a = 0; a < args.argBytes.size(); ++a)
        if (plan.rowBytes[a]) sliced += args.argBytes[a];
      int64_t chunks = std::min<int64_t>(12, std::max<int64_t>(4, static_cast<int64_t>(sliced / (16u << 20))));
      if (const char *forced = std::getenv("AFIR_CUDA_PIPELINE_CHUNKS")) chunks = std::max<int64_t>(2, std::atoll(forced));
      int64_t chunkRows = (plan.rows + chunks - 1) / chunks;
      chunkRows = ((chunkRows + quantum - 1) / quantum) * quantum;
      if (chunkRows < plan.rows) return runHostPipelined(req, *kernel, tiling, args, plan, chunkRows);
    }
  }

  cudaError_t e;
  for (int i = 0; i < req.numInputs; ++i) {
    if (!req.inputBytes[i]) continue;
    if (Status cs = copyToDevice(args.argPtrs[i], req.inputPtrs[i], req.inputBytes[i], stream); !cs) return cs;
    if (launchTraceEnabled()) {
      // what the host handed over, and the same bytes read back from the device (reference
      // NativeExecutionRunner.cpp:391-416: input[i].host, h2d_roundtrip match=..., input[i].h2d_roundtrip)
      const size_t sample = std::min(req.inputBytes[i], kLaunchTraceSampleBytes);
      const unsigned char *host = static_cast<const unsigned char *>(req.inputPtrs[i]);
      printBufferSample("input[" + std::to_string(i) + "].host", host, sample, req.inputBytes[i]);
      unsigned char back[kLaunchTraceSampleBytes] = {0};
      e = cudaMemcpyAsync(back, args.argPtrs[i], sample, cudaMemcpyDeviceToHost, stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] trace read-back failed");
      std::fprintf(stderr, "[cuda-launch] input[%d].h2d_roundtrip match=%s\n", i, std::memcmp(back, host, sample) == 0 ? "yes" : "no");
      printBufferSample("input[" + std::to_string(i) + "].h2d_roundtrip", back, sample, req.inputBytes[i]);
    }
  }
  e = cudaMemsetAsync(workspace_.ptr, 0, kWorkspaceStatusBytes, stream);
  if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] workspace clear failed");

  LaunchInfo info;
  Status ls = dispatch(*kernel, tiling, args, info);
  lastLaunchCount_ = info.kernelsLaunched;
  lastLaunchGenerated_ = info.generated;
  totalLaunchCount_ += static_cast<uint64_t>(info.kernelsLaunched);
  if (!ls) {
    cudaStreamSynchronize(stream);
    return launchStage(ls);
  }
  if (launchTraceEnabled()) std::fprintf(stderr, "[cuda-launch] code=%s kernels=%d\n", info.generated ? "generated" : "library", info.kernelsLaunched);
  if (launchTraceEnabled() && !info.plan.empty()) std::fprintf(stderr, "[cuda-launch] matmul plan: %s\n", info.plan.c_str());
  for (int i = 0; i < req.numOutputs; ++i) {
    if (!req.outputBytes[i]) continue;
    if (Status cs = copyToHost(req.outputPtrs[i], args.argPtrs[req.numInputs + i], req.outputBytes[i], stream); !cs) return cs;
  }
  if (stager_)
    if (Status fs = stager_->finishOut(); !fs) return fs;
  statusPending_ = info.usesStatusBlock;
  statusWorkspace_ = workspace_.ptr;
  matmulPending_ = desc->kernelClass == KernelClass::Matmul;
  reducePending_ = desc->kernelClass == KernelClass::RowReduce;
  Status done = synchronize(stream_);
  if (done && launchTraceEnabled())
    for (int i = 0; i < req.numOutputs; ++i)
      printBufferSample("output[" + std::to_string(i) + "].host_after_d2h", static_cast<const unsigned char *>(req.outputPtrs[i]),
                        std::min(req.outputBytes[i], kLaunchTraceSampleBytes), req.outputBytes[i]);
  Status guards = verifyGuards();
  return done ? guards : done;
}

Status CudaExecutor::ensureCopyStreams(size_t events) {
  cudaError_t e;
  if (!copyIn_) {
    cudaStream_t s;
    if ((e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking)) != cudaSuccess) return cudaFail(e, "cudaStreamCreate");
    copyIn_ = s;
  }
  if (!copyOut_) {
    cudaStream_t s;
    if ((e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking)) != cudaSuccess) return cudaFail(e, "cudaStreamCreate");
    copyOut_ = s;
  }
  while (events_.size() < events) {
    cudaEvent_t ev;
    if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return cudaFail(e, "cudaEventCreate");
    events_.push_back(ev);
  }
  return Status::success();
}

Status CudaExecutor::runHostPipelined(const RunRequest &req, CachedKernel &kernel,
                                      const std::map<std::string, int64_t> &tiling, LaunchArgs &args,
                                      const RowPipelinePlan &plan, int64_t chunkRows) {
  const LaunchDescriptor &desc = *kernel.desc;
  const int64_t numChunks = (plan.rows + chunkRows - 1) / chunkRows;
  if (Status s = ensureCopyStreams(static_cast<size_t>(2 * numChunks + 1)); !s) return s.withStage("cuda:device");
  cudaStream_t compute = static_cast<cudaStream_t>(stream_);
  cudaStream_t in = static_cast<cudaStream_t>(copyIn_);
  cudaStream_t out = static_cast<cudaStream_t>(copyOut_);
  cudaError_t e;
  // `after` starts what it is given next only once everything queued on `before` so far has finished.  A failed
  // record or wait would silently un-order copy and compute, so it ends the run (all three streams drained first).
  auto order = [&](cudaStream_t before, cudaStream_t after, int64_t eventIndex) -> Status {
    cudaEvent_t ev = static_cast<cudaEvent_t>(events_[static_cast<size_t>(eventIndex)]);
    cudaError_t oe = cudaEventRecord(ev, before);
    if (oe == cudaSuccess) oe = cudaStreamWaitEvent(after, ev, 0);
    if (oe == cudaSuccess) return Status::success();
    cudaStreamSynchronize(in);
    cudaStreamSynchronize(compute);
    cudaStreamSynchronize(out);
    return cudaFail(oe, "[cuda:device] ordering the copy and compute streams failed");
  };

  if ((e = cudaMemsetAsync(workspace_.ptr, 0, kWorkspaceStatusBytes, compute)) != cudaSuccess)
    return cudaFail(e, "[cuda:memory] workspace clear failed");
  // arguments every chunk needs in full go first
  for (int i = 0; i < req.numInputs; ++i) {
    if (plan.rowBytes[i] || !req.inputBytes[i]) continue;
    if (Status cs = copyToDevice(args.argPtrs[i], req.inputPtrs[i], req.inputBytes[i], in); !cs) return cs;
  }
  lastLaunchCount_ = 0;
  bool usesStatus = false;
  for (int64_t c = 0; c < numChunks; ++c) {
    const int64_t b = c * chunkRows, en = std::min(plan.rows, b + chunkRows);
    for (int i = 0; i < req.numInputs; ++i) {
      const size_t rb = plan.rowBytes[i];
      if (!rb) continue;
      if (Status cs = copyToDevice(static_cast<char *>(args.argPtrs[i]) + static_cast<size_t>(b) * rb,
                                   static_cast<const char *>(req.inputPtrs[i]) + static_cast<size_t>(b) * rb,
                                   static_cast<size_t>(en - b) * rb, in); !cs)
        return cs;
    }
    if (Status o = order(in, compute, 2 * c); !o) return o;  // the kernel of chunk c waits for its copy-in
    args.rowBegin = b;
    args.rowEnd = en;
    LaunchInfo info;
    Status ls = dispatch(kernel, tiling, args, info);
    lastLaunchCount_ += info.kernelsLaunched;
    lastLaunchGenerated_ = info.generated;
    totalLaunchCount_ += static_cast<uint64_t>(info.kernelsLaunched);
    usesStatus = usesStatus || info.usesStatusBlock;
    if (c == 0 && launchTraceEnabled() && !info.plan.empty())
      std::fprintf(stderr, "[cuda-launch] matmul plan (first of the row chunks): %s\n", info.plan.c_str());
    if (!ls) {
      cudaStreamSynchronize(in);
      cudaStreamSynchronize(compute);
      cudaStreamSynchronize(out);
      return launchStage(ls);
    }
    if (Status o = order(compute, out, 2 * c + 1); !o) return o;  // the copy-out of chunk c waits for its kernel
    for (int i = 0; i < req.numOutputs; ++i) {
      const size_t k = static_cast<size_t>(req.numInputs + i);
      const size_t rb = plan.rowBytes[k];
      if (!rb || !req.outputBytes[i]) continue;
      if (Status cs = copyToHost(static_cast<char *>(req.outputPtrs[i]) + static_cast<size_t>(b) * rb,
                                 static_cast<const char *>(args.argPtrs[k]) + static_cast<size_t>(b) * rb,
                                 static_cast<size_t>(en - b) * rb, out); !cs)
        return cs;
    }
  }
  // outputs that are not row-sliced (none today) would be copied here after the last chunk
  for (int i = 0; i < req.numOutputs; ++i) {
    const size_t k = static_cast<size_t>(req.numInputs + i);
    if (plan.rowBytes[k] || !req.outputBytes[i]) continue;
    if (Status o = order(compute, out, 2 * numChunks); !o) return o;
    if (Status cs = copyToHost(req.outputPtrs[i], args.argPtrs[k], req.outputBytes[i], out); !cs) return cs;
  }
  if (stager_)
    if (Status fs = stager_->finishOut(); !fs) return fs;
  if ((e = cudaStreamSynchronize(in)) != cudaSuccess) return cudaFail(e, "[cuda:memory] host-to-device copy failed");
  if ((e = cudaStreamSynchronize(out)) != cudaSuccess) return cudaFail(e, "[cuda:kernel_launch] kernel execution failed");
  statusPending_ = usesStatus;
  statusWorkspace_ = workspace_.ptr;
  matmulPending_ = desc.kernelClass == KernelClass::Matmul;
  reducePending_ = desc.kernelClass == KernelClass::RowReduce;
  Status done = synchronize(stream_);
  Status guards = verifyGuards();
  return done ? guards : done;
}

Status CudaExecutor::launchDevice(const RunRequest &req, void *workspace, size_t workspaceBytes, void *stream,
                                  const kernels::RowReduceExchange *exchange, const std::vector<const void *> &tableShards,
                                  int64_t rowsPerShard) {
  CachedKernel *kernel = nullptr;
  std::map<std::string, int64_t> tiling;
  if (Status s = validate(req, kernel, tiling); !s) return s;
  const std::shared_ptr<const LaunchDescriptor> desc = kernel->desc;
  cudaError_t e = cudaSetDevice(device_);
  if (e != cudaSuccess) return cudaFail(e, "[cuda:device] cudaSetDevice");

  LaunchArgs args;
  args.device = device_;
  args.stream = static_cast<cudaStream_t>(stream);
  args.blockDim = req.blockDim;
  args.exchange = exchange;
  args.tableShards = tableShards;
  args.rowsPerShard = rowsPerShard;
  for (int i = 0; i < req.numInputs; ++i) {
    args.argPtrs.push_back(const_cast<void *>(req.inputPtrs[i]));
    args.argBytes.push_back(req.inputBytes[i]);
  }
  for (int i = 0; i < req.numOutputs; ++i) {
    args.argPtrs.push_back(req.outputPtrs[i]);
    args.argBytes.push_back(req.outputBytes[i]);
  }
  if (workspace) {
    args.workspace = workspace;
    args.workspaceBytes = workspaceBytes;
  } else {
    size_t wsBytes = 0;
    if (Status s = requiredWorkspaceBytes(*desc, tiling, device_, wsBytes); !s) return s.withStage("cuda:bindings");
    if (Status s = ownWorkspace(wsBytes); !s) return s.withStage("cuda:memory");
    args.workspace = workspace_.ptr;
    args.workspaceBytes = workspace_.capacity;
  }
  if (launchTraceEnabled()) printLaunchTrace(req, *desc, args, device_, "device");
  LaunchInfo info;
  // The status words (bad gather indices, a staged reduction's time-out) accumulate over the launches queued since
  // the last synchronize: they are cleared only when nothing unread is pending on this workspace.
  const bool hasStatusWords = (desc->kernelClass == KernelClass::Gather || desc->kernelClass == KernelClass::RowReduce ||
                               desc->kernelClass == KernelClass::Matmul || desc->kernelClass == KernelClass::Transpose) &&
                              args.workspace && args.workspaceBytes >= kWorkspaceStatusBytes;
  if (hasStatusWords && !(statusPending_ && statusWorkspace_ == args.workspace)) {
    e = cudaMemsetAsync(args.workspace, 0, kWorkspaceStatusReadBytes, args.stream);
    if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] workspace clear failed");
  }
  Status ls = dispatch(*kernel, tiling, args, info);
  lastLaunchCount_ = info.kernelsLaunched;
  lastLaunchGenerated_ = info.generated;
  totalLaunchCount_ += static_cast<uint64_t>(info.kernelsLaunched);
  if (!ls) return launchStage(ls);
  if (launchTraceEnabled() && !info.plan.empty()) std::fprintf(stderr, "[cuda-launch] matmul plan: %s\n", info.plan.c_str());
  if (launchTraceEnabled()) std::fprintf(stderr, "[cuda-launch] code=%s kernels=%d\n", info.generated ? "generated" : "library", info.kernelsLaunched);
  statusPending_ = statusPending_ || info.usesStatusBlock;
  if (info.usesStatusBlock) statusWorkspace_ = args.workspace;
  matmulPending_ = desc->kernelClass == KernelClass::Matmul;
  reducePending_ = desc->kernelClass == KernelClass::RowReduce;
  transposePending_ = transposePending_ || (desc->kernelClass == KernelClass::Transpose && !info.usesStatusBlock);
  return Status::success();
}

Status CudaExecutor::profileResident(const RunRequest &req, int repeats, double &medianMicroseconds) {
  CachedKernel *kernel = nullptr;
  std::map<std::string, int64_t> tiling;
  if (Status s = validate(req, kernel, tiling); !s) return s;
  if (Status s = ensureStream(); !s) return s.withStage("cuda:device");
  const size_t numArgs = static_cast<size_t>(req.numInputs + req.numOutputs);
  if (slots_.size() < numArgs) return Status::error("[cuda:profiling] no resident buffers: run the kernel first");
  LaunchArgs args;
  args.device = device_;
  args.stream = static_cast<cudaStream_t>(stream_);
  args.blockDim = req.blockDim;
  for (int i = 0; i < req.numInputs; ++i) { args.argPtrs.push_back(slots_[i].ptr); args.argBytes.push_back(req.inputBytes[i]); }
  for (int i = 0; i < req.numOutputs; ++i) {
    args.argPtrs.push_back(slots_[req.numInputs + i].ptr);
    args.argBytes.push_back(req.outputBytes[i]);
  }
  args.workspace = workspace_.ptr;
  args.workspaceBytes = workspace_.capacity;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return Status::error("[cuda:profiling] cannot create events");
  std::vector<float> times;
  Status result = Status::success();
  for (int r = 0; r < repeats + 2 && result; ++r) {  // two warm-up launches
    cudaEventRecord(e0, args.stream);
    LaunchInfo info;
    Status ls = dispatch(*kernel, tiling, args, info);
    cudaEventRecord(e1, args.stream);
    totalLaunchCount_ += static_cast<uint64_t>(info.kernelsLaunched);
    if (!ls) { result = ls.withStage("cuda:profiling"); break; }
    if (cudaEventSynchronize(e1) != cudaSuccess) { result = Status::error("[cuda:profiling] kernel execution failed"); break; }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (r >= 2) times.push_back(ms * 1000.0f);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (!result) return result;
  std::sort(times.begin(), times.end());
  medianMicroseconds = times.empty() ? 0.0 : times[times.size() / 2];
  return Status::success();
}

Status CudaExecutor::synchronize(void *stream) {
  if (!initialized_) return Status::error("executor has not been initialized");
  cudaError_t e = cudaSetDevice(device_);
  if (e != cudaSuccess) return cudaFail(e, "[cuda:device] cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream ? stream : stream_);
  e = s ? cudaStreamSynchronize(s) : cudaDeviceSynchronize();
  if (e != cudaSuccess) return cudaFail(e, "[cuda:kernel_launch] kernel execution failed");
  if (statusPending_ && statusWorkspace_) {
    statusPending_ = false;
    unsigned long long words[kWorkspaceStatusReadBytes / 8] = {0, 0, 0};
    e = cudaMemcpy(words, statusWorkspace_, sizeof(words), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cudaFail(e, "[cuda:memory] status read failed");
    const unsigned long long bad = words[0];
    if (static_cast<unsigned int>(words[1] & 0xffffffffull) != 0)
      return Status::error("[cuda:kernel_launch] row reduction: a warp gave up waiting for a bulk copy after 2 s");
    if (const unsigned int mm = static_cast<unsigned int>(words[1] >> 32)) {
      static const char *roles[] = {"TMA producer", "MMA issuer", "epilogue"};
      char text[160];
      std::snprintf(text, sizeof(text), "[cuda:kernel_launch] matmul: %s gave up waiting on a pipeline barrier after 2 s (status 0x%x)",
                    roles[std::min(2u, mm & 0xffu)], mm);
      return Status::error(text);
    }
    if (static_cast<unsigned int>(words[2] & 0xffffffffull) != 0)
      return Status::error("[cuda:kernel_launch] transpose: a wait for a staged tile ran out after 2 s");
    constexpr unsigned long long kGatherTimeoutFlag = 1ull << 62;  // set by the staged gather kernel when a stage wait ran out
    if (bad & kGatherTimeoutFlag) return Status::error("[cuda:kernel_launch] gather kernel gave up waiting for a staged copy");
    if (bad) return Status::error("[cuda:kernel_launch] gather index out of range (" + std::to_string(bad) + " indices)");
  }
  if (reducePending_) {
    reducePending_ = false;
    char text[256] = {0};
    if (kernels::rowReduceCheckStatus(device_, text) != 0)
      return Status::error(std::string("[cuda:kernel_launch] ") + (text[0] ? text : "row reduction reported a wait timeout"));
  }
  if (matmulPending_) {
    matmulPending_ = false;
    char text[256] = {0};
    if (kernels::matmulCheckStatus(device_, text) != 0)
      return Status::error(std::string("[cuda:kernel_launch] ") + (text[0] ? text : "matmul kernel reported a wait timeout"));
  }
  if (transposePending_) {
    transposePending_ = false;
    char text[256] = {0};
    if (kernels::transposeTmaCheckStatus(text, sizeof(text)) != 0)
      return Status::error(std::string("[cuda:kernel_launch] ") + (text[0] ? text : "transpose kernel reported a wait timeout"));
  }
  return Status::success();
}

} // namespace afir
