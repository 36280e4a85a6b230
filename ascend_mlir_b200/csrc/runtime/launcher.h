// Turns a launch descriptor + TilingData values + device pointers into kernel launches.
// Device-side argument order is the reference's canonical kernel signature
// (inputs..., outputs..., workspace, TilingData),
// lib/Conversion/CanonicalizeCannSignature/CanonicalizeCannSignaturePass.cpp:57-140.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "runtime/descriptor.h"

namespace afir {

// Workspace layout: a 256-byte status block (offset 0: u64 count of out-of-range gather indices),
// then kernel scratch (row-reduction partial sums).
constexpr size_t kWorkspaceStatusBytes = 256;

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

} // namespace afir
