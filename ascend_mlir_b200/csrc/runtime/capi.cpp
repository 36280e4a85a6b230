// C entry points (CAPI/Runtime.h, CAPI/RuntimeCuda.h) over CudaExecutor and the descriptor
// "compiler".  Error convention follows the reference (lib/CAPI/Runtime/Runtime.cpp:306-481):
// 0/1 status, message copied (truncated, NUL-terminated) into the caller's buffer on failure only.
#include "CAPI/RuntimeCuda.h"

#include <sys/stat.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iterator>
#include <string>
#include <vector>

#include "execution/artifact_compiler.h"
#include "runtime/caller_device.h"
#include "runtime/executor.h"
#include "runtime/rowsum_exchange.h"

using namespace afir;

#define AFIR_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct CompilerHandle {
  std::string socVersion = "sm_100a";
  std::string arch = "sm_100a";
  int optLevel = 3;
};

void writeErr(char *buf, size_t len, const std::string &msg) {
  if (!buf || len == 0) return;
  std::strncpy(buf, msg.c_str(), len - 1);
  buf[len - 1] = '\0';
}

bool readFile(const std::string &path, std::vector<uint8_t> &out, std::string &err) {
  std::ifstream is(path, std::ios::binary);
  if (!is) { err = "cannot open " + path; return false; }
  out.assign(std::istreambuf_iterator<char>(is), std::istreambuf_iterator<char>());
  if (!is.good() && !is.eof()) { err = "failed reading " + path; return false; }
  return true;
}

bool makeDirs(const std::string &path) {
  std::string cur;
  for (size_t i = 0; i <= path.size(); ++i) {
    if (i == path.size() || path[i] == '/') {
      if (!cur.empty() && ::mkdir(cur.c_str(), 0755) != 0 && errno != EEXIST) return false;
    }
    if (i < path.size()) cur.push_back(path[i]);
  }
  return true;
}

RunRequest makeRequest(const uint8_t *binary, size_t binaryLen, const char *fn, int numInputs, const void **inputPtrs,
                       const size_t *inputBytes, int numOutputs, void **outputPtrs, const size_t *outputBytes,
                       const uint8_t *tiling, size_t tilingLen, int blockDim, uint32_t magic) {
  RunRequest r;
  r.binary = binary;
  r.binaryLen = binaryLen;
  r.functionName = fn ? fn : "";
  r.numInputs = numInputs;
  r.inputPtrs = inputPtrs;
  r.inputBytes = inputBytes;
  r.numOutputs = numOutputs;
  r.outputPtrs = outputPtrs;
  r.outputBytes = outputBytes;
  r.tiling = tiling;
  r.tilingLen = tilingLen;
  r.blockDim = blockDim;
  r.magic = magic;
  return r;
}

} // namespace

AFIR_EXPORT AfirtCompiler afirt_compiler_create(const char *soc_version, const char *arch, int opt_level) {
  auto *h = new (std::nothrow) CompilerHandle();
  if (!h) return nullptr;
  if (soc_version && *soc_version) h->socVersion = soc_version;
  if (arch && *arch) h->arch = arch;
  h->optLevel = opt_level;
  return reinterpret_cast<AfirtCompiler>(h);
}

AFIR_EXPORT void afirt_compiler_destroy(AfirtCompiler compiler) { delete reinterpret_cast<CompilerHandle *>(compiler); }

AFIR_EXPORT int afirt_compiler_compile(AfirtCompiler compiler, const char *src_file, const char *output_dir,
                                       const char *kernel_name, char *out_bin_path, size_t buf_len) {
  auto *h = reinterpret_cast<CompilerHandle *>(compiler);
  if (!h) { writeErr(out_bin_path, buf_len, "compiler handle is null"); return 1; }
  if (!src_file || !*src_file) { writeErr(out_bin_path, buf_len, "kernel source path is required"); return 1; }
  if (!output_dir || !*output_dir) { writeErr(out_bin_path, buf_len, "output directory is required"); return 1; }
  if (!kernel_name || !*kernel_name) { writeErr(out_bin_path, buf_len, "kernel name is required"); return 1; }
  CompileRequest request;
  request.kernelSource = src_file;
  request.outputDir = output_dir;
  request.kernelName = kernel_name;
  request.socVersion = h->socVersion;
  request.arch = h->arch;
  KernelArtifact artifact;
  if (Status s = compileArtifact(request, artifact); !s) { writeErr(out_bin_path, buf_len, s.message()); return 1; }
  const std::string binPath = artifact.deviceBinaryPath;
  writeErr(out_bin_path, buf_len, binPath);
  return 0;
}

AFIR_EXPORT AfirtExecutor afirt_executor_create(void) {
  return reinterpret_cast<AfirtExecutor>(new (std::nothrow) CudaExecutor());
}

AFIR_EXPORT void afirt_executor_destroy(AfirtExecutor executor) {
  CallerDeviceScope keepCallerDevice;
  delete reinterpret_cast<CudaExecutor *>(executor);
}

AFIR_EXPORT int afirt_executor_initialize(AfirtExecutor executor, int device_id, char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex) { writeErr(err_buf, err_len, "executor handle is null"); return 1; }
  if (Status s = ex->initialize(device_id); !s) { writeErr(err_buf, err_len, s.message()); return 1; }
  return 0;
}

AFIR_EXPORT int afirt_executor_run(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                   const char *function_name, int num_inputs, const void **input_ptrs,
                                   const size_t *input_bytes, int num_outputs, void **output_ptrs,
                                   const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                                   int block_dim, uint32_t magic, char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex || !ex->initialized()) { writeErr(err_buf, err_len, "executor has not been initialized"); return 1; }
  if (!binary_data || binary_len == 0) { writeErr(err_buf, err_len, "binary data is required"); return 1; }
  RunRequest r = makeRequest(binary_data, binary_len, function_name, num_inputs, input_ptrs, input_bytes, num_outputs,
                             output_ptrs, output_bytes, tiling_data, tiling_len, block_dim, magic);
  CallerDeviceScope keepCallerDevice;
  if (Status s = ex->runHost(r); !s) { writeErr(err_buf, err_len, s.message()); return 1; }
  return 0;
}

AFIR_EXPORT int afirt_executor_run_file(AfirtExecutor executor, const char *binary_path, const char *function_name,
                                        int num_inputs, const void **input_ptrs, const size_t *input_bytes,
                                        int num_outputs, void **output_ptrs, const size_t *output_bytes,
                                        const uint8_t *tiling_data, size_t tiling_len, int block_dim, uint32_t magic,
                                        char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex || !ex->initialized()) { writeErr(err_buf, err_len, "executor has not been initialized"); return 1; }
  if (!binary_path || !*binary_path) { writeErr(err_buf, err_len, "binary path is required"); return 1; }
  std::vector<uint8_t> bytes;
  std::string err;
  if (!readFile(binary_path, bytes, err)) { writeErr(err_buf, err_len, err); return 1; }
  return afirt_executor_run(executor, bytes.data(), bytes.size(), function_name, num_inputs, input_ptrs, input_bytes,
                            num_outputs, output_ptrs, output_bytes, tiling_data, tiling_len, block_dim, magic, err_buf, err_len);
}

AFIR_EXPORT int afirt_executor_launch_device(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                             const char *function_name, int num_inputs, const void **input_ptrs,
                                             const size_t *input_bytes, int num_outputs, void **output_ptrs,
                                             const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                                             int block_dim, uint32_t magic, void *workspace, size_t workspace_bytes,
                                             void *cuda_stream, char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex || !ex->initialized()) { writeErr(err_buf, err_len, "executor has not been initialized"); return 1; }
  RunRequest r = makeRequest(binary_data, binary_len, function_name, num_inputs, input_ptrs, input_bytes, num_outputs,
                             output_ptrs, output_bytes, tiling_data, tiling_len, block_dim, magic);
  CallerDeviceScope keepCallerDevice;
  if (Status s = ex->launchDevice(r, workspace, workspace_bytes, cuda_stream); !s) {
    writeErr(err_buf, err_len, s.message());
    return 1;
  }
  return 0;
}

AFIR_EXPORT int afirt_executor_launch_device_exchange(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                                      const char *function_name, int num_inputs, const void **input_ptrs,
                                                      const size_t *input_bytes, int num_outputs, void **output_ptrs,
                                                      const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                                                      int block_dim, uint32_t magic, void *workspace, size_t workspace_bytes,
                                                      void *cuda_stream, AfirtRowsumExchange exchange, char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex || !ex->initialized()) { writeErr(err_buf, err_len, "executor has not been initialized"); return 1; }
  kernels::RowReduceExchange record;
  int mailboxDevice = 0;
  if (Status s = nextExchangeCall(exchange, record, mailboxDevice); !s) { writeErr(err_buf, err_len, s.message()); return 1; }
  if (mailboxDevice != ex->device()) { writeErr(err_buf, err_len, "the exchange's mailbox is on another device than the executor"); return 1; }
  RunRequest r = makeRequest(binary_data, binary_len, function_name, num_inputs, input_ptrs, input_bytes, num_outputs,
                             output_ptrs, output_bytes, tiling_data, tiling_len, block_dim, magic);
  CallerDeviceScope keepCallerDevice;
  if (Status s = ex->launchDevice(r, workspace, workspace_bytes, cuda_stream, &record); !s) {
    writeErr(err_buf, err_len, s.message());
    return 1;
  }
  commitExchangeCall(exchange, record);
  return 0;
}

AFIR_EXPORT int afirt_executor_launch_device_sharded_table(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                                           const char *function_name, int num_inputs, const void **input_ptrs,
                                                           const size_t *input_bytes, int num_outputs, void **output_ptrs,
                                                           const size_t *output_bytes, const uint8_t *tiling_data, size_t tiling_len,
                                                           int block_dim, uint32_t magic, void *workspace, size_t workspace_bytes,
                                                           void *cuda_stream, int num_shards, const void **shard_ptrs,
                                                           int64_t rows_per_shard, char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex || !ex->initialized()) { writeErr(err_buf, err_len, "executor has not been initialized"); return 1; }
  if (num_shards < 1 || !shard_ptrs) { writeErr(err_buf, err_len, "at least one table shard is required"); return 1; }
  if (rows_per_shard < 1) { writeErr(err_buf, err_len, "rows_per_shard must be positive"); return 1; }
  std::vector<const void *> shards(shard_ptrs, shard_ptrs + num_shards);
  RunRequest r = makeRequest(binary_data, binary_len, function_name, num_inputs, input_ptrs, input_bytes, num_outputs,
                             output_ptrs, output_bytes, tiling_data, tiling_len, block_dim, magic);
  CallerDeviceScope keepCallerDevice;
  if (Status s = ex->launchDevice(r, workspace, workspace_bytes, cuda_stream, nullptr, shards, rows_per_shard); !s) {
    writeErr(err_buf, err_len, s.message());
    return 1;
  }
  return 0;
}

AFIR_EXPORT int afirt_executor_synchronize(AfirtExecutor executor, void *cuda_stream, char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex || !ex->initialized()) { writeErr(err_buf, err_len, "executor has not been initialized"); return 1; }
  CallerDeviceScope keepCallerDevice;
  if (Status s = ex->synchronize(cuda_stream); !s) { writeErr(err_buf, err_len, s.message()); return 1; }
  return 0;
}

AFIR_EXPORT int afirt_executor_workspace_bytes(AfirtExecutor executor, const uint8_t *binary_data, size_t binary_len,
                                               const uint8_t *tiling_data, size_t tiling_len, size_t *out_bytes,
                                               char *err_buf, size_t err_len) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  if (!ex || !ex->initialized()) { writeErr(err_buf, err_len, "executor has not been initialized"); return 1; }
  if (!out_bytes) { writeErr(err_buf, err_len, "out_bytes is required"); return 1; }
  LaunchDescriptor desc;
  if (Status s = parseDescriptorBinary(binary_data, binary_len, desc); !s) { writeErr(err_buf, err_len, s.message()); return 1; }
  std::map<std::string, int64_t> tiling;
  if (Status s = unpackTiling(desc, tiling_data, tiling_len, tiling); !s) { writeErr(err_buf, err_len, s.message()); return 1; }
  size_t bytes = 0;
  CallerDeviceScope keepCallerDevice;
  if (Status s = requiredWorkspaceBytes(desc, tiling, ex->device(), bytes); !s) { writeErr(err_buf, err_len, s.message()); return 1; }
  *out_bytes = bytes;
  return 0;
}

AFIR_EXPORT int afirt_executor_last_launch_count(AfirtExecutor executor) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  return ex ? ex->lastLaunchCount() : 0;
}

AFIR_EXPORT int afirt_executor_last_launch_generated(AfirtExecutor executor) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  return ex && ex->lastLaunchGenerated() ? 1 : 0;
}

AFIR_EXPORT uint64_t afirt_executor_total_launch_count(AfirtExecutor executor) {
  auto *ex = reinterpret_cast<CudaExecutor *>(executor);
  return ex ? ex->totalLaunchCount() : 0;
}

AFIR_EXPORT const char *afirt_runtime_version(void) { return "afir-b200 0.1 sm_100a"; }
