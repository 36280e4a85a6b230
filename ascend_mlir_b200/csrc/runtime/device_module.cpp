#include "runtime/device_module.h"

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdlib>
#include <mutex>

namespace afir {
namespace {

struct DriverApi {
  std::string reason;
  decltype(&cuModuleLoadData) moduleLoadData = nullptr;
  decltype(&cuModuleUnload) moduleUnload = nullptr;
  decltype(&cuModuleGetFunction) moduleGetFunction = nullptr;
  decltype(&cuLaunchKernel) launchKernel = nullptr;
  decltype(&cuLaunchKernelEx) launchKernelEx = nullptr;  // optional: programmatic dependent launch
  bool dependentLaunch = false;
  decltype(&cuFuncSetAttribute) funcSetAttribute = nullptr;
  decltype(&cuGetErrorString) getErrorString = nullptr;
};

const DriverApi &driver() {
  static DriverApi d;
  static std::once_flag once;
  std::call_once(once, [] {
    auto resolve = [&](const char *name, auto &fn) {
      void *p = nullptr;
      cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
      const cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &found);
      if (e != cudaSuccess || found != cudaDriverEntryPointSuccess || !p) {
        if (d.reason.empty()) d.reason = std::string("the CUDA driver has no entry point ") + name;
        return;
      }
      fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(p);
    };
    resolve("cuModuleLoadData", d.moduleLoadData);
    resolve("cuModuleUnload", d.moduleUnload);
    resolve("cuModuleGetFunction", d.moduleGetFunction);
    resolve("cuLaunchKernel", d.launchKernel);
    resolve("cuFuncSetAttribute", d.funcSetAttribute);
    resolve("cuGetErrorString", d.getErrorString);
    {  // optional entry point: its absence only turns programmatic dependent launch off
      const std::string keep = d.reason;
      resolve("cuLaunchKernelEx", d.launchKernelEx);
      d.reason = keep;
      const char *pdl = std::getenv("AFIR_CUDA_PDL");
      d.dependentLaunch = d.launchKernelEx != nullptr && !(pdl && pdl[0] == '0');
    }
  });
  return d;
}

Status driverError(const DriverApi &d, CUresult r, const std::string &what) {
  const char *text = nullptr;
  if (d.getErrorString) d.getErrorString(r, &text);
  return Status::error(what + ": " + (text ? text : "CUDA driver error " + std::to_string(static_cast<int>(r))));
}

} // namespace

DeviceModule::~DeviceModule() {
  // Unloading needs the owning context; at process exit it may already be gone, which the driver reports and
  // which needs no handling.
  const DriverApi &d = driver();
  if (module_ && d.moduleUnload && cudaSetDevice(device_) == cudaSuccess) d.moduleUnload(static_cast<CUmodule>(module_));
}

Status DeviceModule::load(const void *cubin, size_t bytes, int device, std::shared_ptr<DeviceModule> &out) {
  if (!cubin || bytes == 0) return Status::error("empty device binary");
  const DriverApi &d = driver();
  if (!d.reason.empty()) return Status::error(d.reason);
  // The runtime creates the device's primary context on first use and makes it current on this thread.
  cudaError_t e = cudaFree(nullptr);
  if (e != cudaSuccess) return Status::error(std::string("cannot initialise the device context: ") + cudaGetErrorString(e));
  CUmodule m = nullptr;
  const CUresult r = d.moduleLoadData(&m, cubin);
  if (r != CUDA_SUCCESS) return driverError(d, r, "cuModuleLoadData");
  out.reset(new DeviceModule());
  out->module_ = m;
  out->device_ = device;
  return Status::success();
}

Status DeviceModule::function(const std::string &name, void *&fn) {
  auto it = functions_.find(name);
  if (it != functions_.end()) { fn = it->second; return Status::success(); }
  const DriverApi &d = driver();
  CUfunction f = nullptr;
  const CUresult r = d.moduleGetFunction(&f, static_cast<CUmodule>(module_), name.c_str());
  if (r != CUDA_SUCCESS) return driverError(d, r, "cuModuleGetFunction(" + name + ")");
  functions_[name] = f;
  fn = f;
  return Status::success();
}

Status DeviceModule::reserveDynamicSharedMemory(void *fn, int bytes) {
  auto it = reserved_.find(fn);
  if (it != reserved_.end() && it->second >= bytes) return Status::success();
  const DriverApi &d = driver();
  const CUresult r = d.funcSetAttribute(static_cast<CUfunction>(fn), CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, bytes);
  if (r != CUDA_SUCCESS) return driverError(d, r, "cuFuncSetAttribute(max dynamic shared memory)");
  reserved_[fn] = bytes;
  return Status::success();
}

Status launchDeviceFunction(void *fn, unsigned int grid, unsigned int block, size_t dynamicSmemBytes, cudaStream_t stream,
                            void **params, bool waitsForDependencies) {
  const DriverApi &d = driver();
  if (!d.reason.empty()) return Status::error(d.reason);
  if (d.dependentLaunch && waitsForDependencies) {
    // Generated kernels begin with gridDependencyPrologue(): launched with programmatic stream serialisation their
    // CTAs are scheduled while the previous kernel of the stream drains, and wait there for it to complete.
    CUlaunchAttribute attr;
    attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr.value.programmaticStreamSerializationAllowed = 1;
    CUlaunchConfig cfg = {};
    cfg.gridDimX = grid; cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = block; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = static_cast<unsigned int>(dynamicSmemBytes);
    cfg.hStream = reinterpret_cast<CUstream>(stream);
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const CUresult r = d.launchKernelEx(&cfg, static_cast<CUfunction>(fn), params, nullptr);
    if (r != CUDA_SUCCESS) return driverError(d, r, "cuLaunchKernelEx");
    return Status::success();
  }
  const CUresult r = d.launchKernel(static_cast<CUfunction>(fn), grid, 1, 1, block, 1, 1, static_cast<unsigned int>(dynamicSmemBytes),
                                    reinterpret_cast<CUstream>(stream), params, nullptr);
  if (r != CUDA_SUCCESS) return driverError(d, r, "cuLaunchKernel");
  return Status::success();
}

} // namespace afir
