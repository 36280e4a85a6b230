// Generated device binaries on the GPU: load a cubin, look a kernel up by name, launch it.  The reference's runner
// does the same with its runtime's register/launch calls and caches by (path, name, magic)
// (lib/Runtime/Execution/NativeExecutionRunner.cpp:223,332,476); here the calls are the CUDA driver API's
// cuModuleLoadData / cuModuleGetFunction / cuLaunchKernel, resolved through the CUDA runtime
// (cudaGetDriverEntryPoint) so that the library links against no driver stub and shares the runtime's primary
// context with the prebuilt kernels.
#pragma once

#include <cstddef>
#include <map>
#include <memory>
#include <string>

#include "common/status.h"

typedef struct CUstream_st *cudaStream_t;

namespace afir {

class DeviceModule {
public:
  ~DeviceModule();
  DeviceModule(const DeviceModule &) = delete;
  DeviceModule &operator=(const DeviceModule &) = delete;

  // Loads `cubin` into the current device's primary context (the caller has made the device current).
  static Status load(const void *cubin, size_t bytes, int device, std::shared_ptr<DeviceModule> &out);
  // The kernel named `name` (cached); error when the module has none.
  Status function(const std::string &name, void *&fn);
  // Opts `fn` into `bytes` of dynamic shared memory (beyond the 48 KB every kernel may use).
  Status reserveDynamicSharedMemory(void *fn, int bytes);

private:
  DeviceModule() = default;
  void *module_ = nullptr;
  int device_ = 0;
  std::map<std::string, void *> functions_;
  std::map<void *, int> reserved_;
};

// cuLaunchKernel: a 1-D grid of `grid` CTAs of `block` threads; params[i] points at the i-th kernel argument.
// `waitsForDependencies`: the kernel begins with gridDependencyPrologue(), so it may be launched with programmatic
// stream serialisation (cuLaunchKernelEx; AFIR_CUDA_PDL=0 turns that off) and start up under the previous kernel's tail.
Status launchDeviceFunction(void *fn, unsigned int grid, unsigned int block, size_t dynamicSmemBytes, cudaStream_t stream,
                            void **params, bool waitsForDependencies = false);

} // namespace afir
