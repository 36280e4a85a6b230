#include "runtime/caller_device.h"

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <mutex>

namespace afir {
namespace {

decltype(&cuCtxGetCurrent) contextGetter() {
  static decltype(&cuCtxGetCurrent) fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &found) == cudaSuccess &&
        found == cudaDriverEntryPointSuccess && p)
      fn = reinterpret_cast<decltype(&cuCtxGetCurrent)>(p);
  });
  return fn;
}

} // namespace

CallerDeviceScope::CallerDeviceScope() {
  auto getCurrent = contextGetter();
  CUcontext ctx = nullptr;
  if (!getCurrent || getCurrent(&ctx) != CUDA_SUCCESS || !ctx) return;  // nothing current: nothing to put back
  int device = -1;
  if (cudaGetDevice(&device) == cudaSuccess) previous_ = device;
}

CallerDeviceScope::~CallerDeviceScope() {
  if (previous_ < 0) return;
  int now = -1;
  if (cudaGetDevice(&now) == cudaSuccess && now != previous_) cudaSetDevice(previous_);
}

} // namespace afir
