// Turns a launch descriptor + TilingData values + device pointers into kernel launches.
// Device-side argument order is the reference's canonical kernel signature
// (inputs..., outputs..., workspace, TilingData),
// lib/Conversion/CanonicalizeCannSignature/CanonicalizeCannSignaturePass.cpp:57-140.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "runtime/descriptor.h"
#include "runtime/device_module.h"

namespace afir {

// Workspace layout: a 256-byte status block (offset 0: u64 count of out-of-range gather indices, offset 8: u32
// time-out flag of the staged row-reduction kernel, offset 12: u32 time-out word of the matmul kernel), then kernel
// scratch (row-reduction partial sums).
constexpr size_t kWorkspaceStatusBytes = 256;
constexpr size_t kWorkspaceReduceStatusOffset = 8;  // u32: a staged row-reduction kernel gave up waiting for a copy
constexpr size_t kWorkspaceMatmulStatusOffset = 12; // u32: (1 << 8) | role of a matmul pipeline wait that ran out
constexpr size_t kWorkspaceTransposeStatusOffset = 16;  // u32: the copy-engine transpose gave up waiting for a tile
constexpr size_t kWorkspaceStatusReadBytes = 24;    // what the executor reads back after a run

struct LaunchArgs {
  std::vector<void *> argPtrs;  // device pointers, inputs first then outputs
  std::vector<size_t> argBytes;
  void *workspace = nullptr;
  size_t workspaceBytes = 0;
  int blockDim = 0;  // CTAs to launch; <= 0 lets the library choose
  // Optional sub-range [rowBegin, rowEnd) of the leading iteration dim (single-group descriptors and
  // matmul rows); rowEnd < 0 = everything.  Used to pipeline host copies with compute.
  int64_t rowBegin = 0;
  int64_t rowEnd = -1;
  cudaStream_t stream = nullptr;
  int device = 0;
  // Row-reduction groups only: the reduced axis is sharded over GPUs and the kernel exchanges its partial sums
  // through this mailbox record (see kernels::RowReduceExchange); null = an ordinary launch.
  const kernels::RowReduceExchange *exchange = nullptr;
  // Row-gather groups only: the table argument is given as row shards instead (possibly other GPUs' memory,
  // peer-mapped).  Its entry in argPtrs is ignored (may be null); its entry in argBytes is the whole table's size.
  std::vector<const void *> tableShards;
  int64_t rowsPerShard = 0;
};

struct LaunchInfo {
  int kernelsLaunched = 0;
  bool usesStatusBlock = false;  // caller should zero it before and check it after
  bool generated = false;        // the launch ran the group's generated kernel, not a prebuilt one
  std::string plan;              // matmul: the planner's one-line description of what was launched
};

// Scratch bytes (status block included) the descriptor needs at these tiling values.
Status requiredWorkspaceBytes(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, int device,
                              size_t &bytes);

// How the host path may cut a run into leading-axis chunks: `rows` is the leading extent and, per
// kernel argument, rowBytes > 0 means "rows [b, e) of the work touch bytes [b*rowBytes, e*rowBytes) of
// this argument", 0 means the whole argument is needed by every chunk.  possible = false when the
// descriptor cannot be chunked (several groups, permuted leading dims, sliced views).
struct RowPipelinePlan {
  bool possible = false;
  int64_t rows = 0;
  std::vector<size_t> rowBytes;
};
Status planRowPipeline(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling,
                       const std::vector<size_t> &argBytes, RowPipelinePlan &plan);

Status launchDescriptor(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args,
                        LaunchInfo &info);

// ---- generated kernels -------------------------------------------------------------------------------------------
// The kernel generated for one descriptor (codegen/kernel_source), loaded on one device.
struct GeneratedBinding {
  std::shared_ptr<DeviceModule> module;
  void *mainFn = nullptr;      // <kernel>
  void *stagedFn = nullptr;    // <kernel>__staged (row reductions with one streamed view), or null
  void *finalizeFn = nullptr;  // <kernel>__finalize (row reductions), or null
  void *singleVectorFn = nullptr;  // <kernel>__one (row gathers: one vector per thread in flight), or null
  bool ctasOf256Threads = false;  // elementwise: the kernel holds the register-block loop and is compiled for CTAs of 256 threads
  bool waitsForDependencies = false;  // every entry begins with gridDependencyPrologue() (the module says so by a marker kernel)
};

// True when this launch can run on the descriptor's generated kernel: the features the generated code does not
// cover (an exchange of partial sums between GPUs, a sharded gather table, a tuning value of the prebuilt
// kernels' unroll or staged-copy options) stay on the library's kernels.
bool generatedLaunchApplies(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args);

// Same contract as launchDescriptor, on the generated kernel: same checks of sizes and bounds, same launch plan,
// the kernel arguments in the reference's order (inputs..., outputs..., workspace, TilingData).
Status launchGenerated(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args,
                       GeneratedBinding &binding, LaunchInfo &info);

} // namespace afir
