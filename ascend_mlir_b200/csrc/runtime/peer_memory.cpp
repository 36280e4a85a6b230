// afirt_peer_*: device memory of one process made addressable from another process's GPU (CUDA IPC), for operands
// that live on other GPUs of the node: the row shards of a gather table, for instance.  Thin, but with the two
// things raw cudaIpc* leaves to the caller: a pointer INSIDE an allocation can be exported (frameworks hand out
// sub-allocations of large blocks; the handle then carries the offset), and importing the same allocation twice in
// one process shares one mapping (the driver refuses a second cudaIpcOpenMemHandle of an open handle).
#include "CAPI/RuntimeCuda.h"

#include <cuda.h>
#include "runtime/caller_device.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unistd.h>

namespace {

struct PeerHandle {  // AFIRT_PEER_HANDLE_BYTES
  cudaIpcMemHandle_t ipc;  // 64 bytes: the whole allocation
  uint64_t offset;         // of the exported pointer inside it
  uint64_t pid;            // exporter (a process cannot import its own memory: it already has it)
  uint64_t address;        // exporter's pointer, returned as it is inside the exporting process
  int32_t device;
  int32_t reserved;
};
static_assert(sizeof(PeerHandle) == AFIRT_PEER_HANDLE_BYTES, "peer handle layout");

struct Mapping { void *base = nullptr; int refs = 0; };
std::mutex g_mu;
std::map<std::string, Mapping> g_byHandle;   // key: the 64 ipc bytes
struct Handout { std::string key; int count = 0; };
std::map<void *, Handout> g_byPointer;       // pointer handed out -> its mapping, and how many imports returned it

void fail(char *buf, size_t len, const char *what, cudaError_t e = cudaSuccess) {
  if (!buf || len == 0) return;
  if (e != cudaSuccess) std::snprintf(buf, len, "%s: %s", what, cudaGetErrorString(e));
  else std::snprintf(buf, len, "%s", what);
}

using GetAddressRangeFn = CUresult (*)(CUdeviceptr *, size_t *, CUdeviceptr);
GetAddressRangeFn addressRangeFn() {
  static GetAddressRangeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<GetAddressRangeFn>(p);
  }();
  return fn;
}

} // namespace

#define AFIRT_EXPORT extern "C" __attribute__((visibility("default")))

AFIRT_EXPORT int afirt_peer_export(const void *device_ptr, uint8_t *out_handle, char *err_buf, size_t err_len) {
  if (!device_ptr || !out_handle) { fail(err_buf, err_len, "device_ptr and out_handle are required"); return 1; }
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, device_ptr);
  if (e != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
    (void)cudaGetLastError();
    fail(err_buf, err_len, "afirt_peer_export: not a device pointer");
    return 1;
  }
  afir::CallerDeviceScope keepCallerDevice;
  e = cudaSetDevice(attr.device);
  if (e != cudaSuccess) { fail(err_buf, err_len, "cudaSetDevice", e); return 1; }
  GetAddressRangeFn range = addressRangeFn();
  CUdeviceptr base = 0;
  size_t size = 0;
  if (!range || range(&base, &size, reinterpret_cast<CUdeviceptr>(device_ptr)) != CUDA_SUCCESS) {
    fail(err_buf, err_len, "afirt_peer_export: cannot find the allocation that holds the pointer");
    return 1;
  }
  PeerHandle h;
  std::memset(&h, 0, sizeof(h));
  e = cudaIpcGetMemHandle(&h.ipc, reinterpret_cast<void *>(base));
  if (e != cudaSuccess) { fail(err_buf, err_len, "cudaIpcGetMemHandle (memory from cudaMalloc is required)", e); return 1; }
  h.offset = reinterpret_cast<uint64_t>(device_ptr) - static_cast<uint64_t>(base);
  h.pid = static_cast<uint64_t>(getpid());
  h.address = reinterpret_cast<uint64_t>(device_ptr);
  h.device = attr.device;
  std::memcpy(out_handle, &h, sizeof(h));
  return 0;
}

AFIRT_EXPORT int afirt_peer_import(int device_id, const uint8_t *handle, void **out_ptr, char *err_buf, size_t err_len) {
  if (!handle || !out_ptr) { fail(err_buf, err_len, "handle and out_ptr are required"); return 1; }
  *out_ptr = nullptr;
  PeerHandle h;
  std::memcpy(&h, handle, sizeof(h));
  afir::CallerDeviceScope keepCallerDevice;
  cudaError_t e = cudaSetDevice(device_id);
  if (e != cudaSuccess) { fail(err_buf, err_len, "cudaSetDevice", e); return 1; }
  if (h.pid == static_cast<uint64_t>(getpid())) {
    // the exporter's own process: the pointer is valid here; another device of this process needs peer access
    if (h.device != device_id) {
      int can = 0;
      e = cudaDeviceCanAccessPeer(&can, device_id, h.device);
      if (e == cudaSuccess && !can) { fail(err_buf, err_len, "no peer access between the two devices"); return 1; }
      if (e == cudaSuccess) {
        e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) { e = cudaSuccess; (void)cudaGetLastError(); }
      }
      if (e != cudaSuccess) { fail(err_buf, err_len, "enabling peer access", e); return 1; }
    }
    *out_ptr = reinterpret_cast<void *>(h.address);
    return 0;
  }
  const std::string key(reinterpret_cast<const char *>(&h.ipc), sizeof(h.ipc));
  std::lock_guard<std::mutex> lock(g_mu);
  Mapping &m = g_byHandle[key];
  if (!m.base) {
    e = cudaIpcOpenMemHandle(&m.base, h.ipc, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      g_byHandle.erase(key);
      fail(err_buf, err_len, "cudaIpcOpenMemHandle", e);
      return 1;
    }
  }
  ++m.refs;
  void *p = static_cast<char *>(m.base) + h.offset;
  Handout &out = g_byPointer[p];
  out.key = key;
  ++out.count;
  *out_ptr = p;
  return 0;
}

AFIRT_EXPORT int afirt_peer_release(void *imported_ptr, char *err_buf, size_t err_len) {
  if (!imported_ptr) return 0;
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_byPointer.find(imported_ptr);
  if (it == g_byPointer.end()) return 0;  // a pointer of this process's own memory: nothing was mapped
  const std::string key = it->second.key;
  if (--it->second.count <= 0) g_byPointer.erase(it);
  auto mt = g_byHandle.find(key);
  if (mt != g_byHandle.end() && --mt->second.refs <= 0) {  // the last pointer into this allocation: unmap it
    cudaError_t e = cudaIpcCloseMemHandle(mt->second.base);
    g_byHandle.erase(mt);
    if (e != cudaSuccess) { fail(err_buf, err_len, "cudaIpcCloseMemHandle", e); return 1; }
  }
  return 0;
}
