// Host side of programmatic dependent launch for the library's own kernels.  A kernel that begins with
// gridDependencyPrologue() (kernels/grid_dependency.cuh) is launched through launchDependent(): its CTAs are
// scheduled while the previous kernel of the stream is draining and wait there until that kernel has completed, so
// the stream's order is unchanged and a launch's start-up cost is hidden behind its predecessor's tail.
// AFIR_CUDA_PDL=0 turns the attribute off (the kernels' prologue then does nothing).
//
// Which kernels: the elementwise, row-reduction and transpose kernels (measured gain 0.3-1 us per launch, up to
// 8 % on a 8 us launch).  Not the gather kernels: their grid is one CTA per tile, tens of thousands of short CTAs,
// and the two prologue instructions in every CTA cost the cfg4 gather 7 us of 62 (measured with and without, same
// GPU).  Not the matmul either: its CTAs fill an SM's shared memory, so a dependent CTA cannot become resident
// before its predecessor's CTA has gone, and there is nothing to overlap.  Those two use launchOrdinary().
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace afir {
namespace kernels {

inline bool dependentLaunchEnabled() {
  static const bool on = [] {
    const char *v = std::getenv("AFIR_CUDA_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

template <class... Params, class... Args>
cudaError_t launchDependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t dynamicSmemBytes, cudaStream_t stream,
                            Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = dynamicSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependentLaunchEnabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <class... Params, class... Args>
cudaError_t launchOrdinary(void (*kernel)(Params...), dim3 grid, dim3 block, size_t dynamicSmemBytes, cudaStream_t stream,
                           Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = dynamicSmemBytes;
  cfg.stream = stream;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

} // namespace kernels
} // namespace afir
