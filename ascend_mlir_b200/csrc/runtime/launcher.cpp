#include "runtime/launcher.h"
#include "kernels/matmul_plan.h"

#include <algorithm>
#include <cstring>

namespace afir {
namespace {

Status evalDim(const DimExpr &e, const std::map<std::string, int64_t> &tiling, int64_t &out) {
  if (e.literal) { out = e.value; return Status::success(); }
  auto it = tiling.find(e.field);
  if (it == tiling.end()) return Status::error("tiling field '" + e.field + "' is not in the kernel's TilingData");
  out = it->second;
  if (out < 0) return Status::error("tiling field '" + e.field + "' is negative");
  return Status::success();
}

Status evalDims(const std::vector<DimExpr> &es, const std::map<std::string, int64_t> &tiling, std::vector<int64_t> &out) {
  out.resize(es.size());
  for (size_t i = 0; i < es.size(); ++i)
    if (Status s = evalDim(es[i], tiling, out[i]); !s) return s;
  return Status::success();
}

int64_t optionalField(const std::string &name, const std::map<std::string, int64_t> &tiling) {
  if (name.empty()) return 0;
  auto it = tiling.find(name);
  return it == tiling.end() ? 0 : it->second;
}

int toElemType(DType t, bool &ok, bool integersToo = false) {
  ok = true;
  switch (t) {
  case DType::F32: return kernels::kF32;
  case DType::F16: return kernels::kF16;
  case DType::BF16: return kernels::kBF16;
  case DType::I32: ok = integersToo; return kernels::kInt32;
  case DType::I16: ok = integersToo; return kernels::kInt16;
  default: ok = false; return 0;
  }
}

// A view resolved against concrete sizes: element strides per iteration dim and a base offset.
struct ResolvedView {
  int arg = -1;
  size_t elemBytes = 0;
  int64_t baseOffset = 0;       // elements
  std::vector<int64_t> stride;  // per domain dim
};

Status resolveView(const ViewSpec &v, const std::vector<int64_t> &domain, const std::map<std::string, int64_t> &tiling,
                   const LaunchArgs &args, const char *what, ResolvedView &out) {
  std::vector<int64_t> shape, offset;
  if (Status s = evalDims(v.shape, tiling, shape); !s) return s;
  if (v.offset.empty()) offset.assign(shape.size(), 0);
  else if (Status s = evalDims(v.offset, tiling, offset); !s) return s;
  out.arg = v.arg;
  out.elemBytes = dtypeBytes(v.dtype);
  int64_t elems = 1;
  for (int64_t d : shape) elems *= d;
  const size_t want = static_cast<size_t>(elems) * out.elemBytes;
  if (v.arg >= static_cast<int>(args.argBytes.size())) return Status::error(std::string(what) + ": argument index out of range");
  if (args.argBytes[v.arg] != want)
    return Status::error("[cuda:bindings] " + std::string(what) + ": argument " + std::to_string(v.arg) + " is " +
                         std::to_string(args.argBytes[v.arg]) + " bytes, the tiling dims imply " + std::to_string(want));
  out.stride.assign(domain.size(), 0);
  out.baseOffset = 0;
  int64_t ts = 1;
  for (int t = static_cast<int>(shape.size()) - 1; t >= 0; --t) {
    const int d = v.map.empty() ? -1 : v.map[t];
    const int64_t extent = d >= 0 ? domain[d] : 1;
    if (d == 0 && args.rowEnd >= 0) offset[t] += args.rowBegin;
    if (offset[t] < 0 || offset[t] + extent > shape[t])
      return Status::error(std::string(what) + ": view exceeds argument " + std::to_string(v.arg) + " along dim " + std::to_string(t));
    if (d >= 0) out.stride[d] += ts;
    out.baseOffset += offset[t] * ts;
    ts *= shape[t];
  }
  return Status::success();
}

// Collapses the iteration space: drops extent-1 dims and merges neighbours that every view walks
// contiguously (a broadcast view, stride 0 on both, merges too).  Strides are rewritten in place.
void collapseDomain(std::vector<int64_t> &domain, std::vector<ResolvedView *> &views) {
  for (size_t d = 0; d < domain.size() && domain.size() > 1;) {
    if (domain[d] == 1) {
      domain.erase(domain.begin() + d);
      for (auto *v : views) v->stride.erase(v->stride.begin() + d);
    } else ++d;
  }
  for (size_t d = 0; d + 1 < domain.size();) {
    bool mergeable = true;
    for (auto *v : views)
      if (v->stride[d] != v->stride[d + 1] * domain[d + 1]) { mergeable = false; break; }
    if (mergeable) {
      domain[d + 1] *= domain[d];
      domain.erase(domain.begin() + d);
      for (auto *v : views) v->stride.erase(v->stride.begin() + d);
    } else ++d;
  }
}

// Restricts the leading iteration dim to the requested row range (no-op when none was asked for).
Status applyRowRange(std::vector<int64_t> &domain, const LaunchArgs &args, int64_t *fullRows = nullptr) {
  if (fullRows) *fullRows = domain.empty() ? 0 : domain[0];
  if (args.rowEnd < 0) return Status::success();
  if (domain.empty() || args.rowBegin < 0 || args.rowBegin > args.rowEnd || args.rowEnd > domain[0])
    return Status::error("row range outside the leading iteration dim");
  domain[0] = args.rowEnd - args.rowBegin;
  return Status::success();
}

void *argAt(const LaunchArgs &args, const ResolvedView &v) {
  return static_cast<char *>(args.argPtrs[v.arg]) + static_cast<size_t>(v.baseOffset) * v.elemBytes;
}

Status cudaStatus(int code, const char *what) {
  if (code == 0) return Status::success();
  return Status::error(std::string(what) + ": " + kernels::cudaErrorText(code));
}

// Evaluates an elementwise group's domain and views at these tiling values and checks every argument's size and
// every view's bounds (shared by the prebuilt and the generated launch).
Status resolveElementwiseGroup(const LaunchDescriptor &d, const GroupSpec &g, const std::map<std::string, int64_t> &tiling,
                               const LaunchArgs &args, int &et, std::vector<int64_t> &domain, std::vector<ResolvedView> &loads,
                               ResolvedView &store) {
  bool ok;
  et = toElemType(d.dtype, ok, /*integersToo=*/true);
  if (!ok) return Status::error("elementwise groups compute in f32, f16, bf16, i32 or i16");
  if (Status s = evalDims(g.domain, tiling, domain); !s) return s;
  if (Status s = applyRowRange(domain, args); !s) return s;
  loads.assign(g.loads.size(), ResolvedView());
  for (size_t i = 0; i < g.loads.size(); ++i) {
    if (g.loads[i].dtype != d.dtype) return Status::error("load " + std::to_string(i) + " differs from the group element type");
    if (Status s = resolveView(g.loads[i], domain, tiling, args, "load", loads[i]); !s) return s;
  }
  return resolveView(g.store, domain, tiling, args, "store", store);
}

Status launchElementwiseGroup(const LaunchDescriptor &d, const GroupSpec &g, const std::map<std::string, int64_t> &tiling,
                              const LaunchArgs &args, LaunchInfo &info) {
  int et = 0;
  std::vector<int64_t> domain;
  std::vector<ResolvedView> loads;
  ResolvedView store;
  if (Status s = resolveElementwiseGroup(d, g, tiling, args, et, domain, loads, store); !s) return s;
  std::vector<ResolvedView *> all;
  for (auto &v : loads) all.push_back(&v);
  all.push_back(&store);
  collapseDomain(domain, all);
  // The kernels walk three dims.  What is left above them after collapsing (a permutation of rank four or more
  // that no merge simplifies) is walked here, one launch per index of those outer dims.
  constexpr int64_t kMaxOuterLaunches = 4096;
  std::vector<int64_t> outer;
  std::vector<std::vector<int64_t>> outerStride(all.size());
  while (domain.size() > 3) {
    outer.push_back(domain.front());
    domain.erase(domain.begin());
    for (size_t i = 0; i < all.size(); ++i) {
      outerStride[i].push_back(all[i]->stride.front());
      all[i]->stride.erase(all[i]->stride.begin());
    }
  }
  int64_t outerCount = 1;
  for (size_t j = 0; j < outer.size(); ++j) {
    outerCount *= outer[j];
    if (j + 1 < outer.size() && outerCount > kMaxOuterLaunches)  // the last of them is not walked here (below)
      return Status::error("iteration space keeps more than three dims after collapsing and the outer ones need more than " +
                           std::to_string(kMaxOuterLaunches) + " launches");
  }
  while (domain.size() < 3) {
    domain.insert(domain.begin(), 1);
    for (auto *v : all) v->stride.insert(v->stride.begin(), 0);
  }
  if (store.stride[2] != 1 && domain[2] != 1) return Status::error("the store must be contiguous along the inner dim");

  kernels::ElementwiseLaunch l = {};
  l.elemType = et;
  for (int i = 0; i < 3; ++i) l.dims[i] = domain[i];
  l.numViews = static_cast<int>(loads.size());
  for (size_t i = 0; i < loads.size(); ++i) {
    for (int k = 0; k < 3; ++k) l.views[i].stride[k] = loads[i].stride[k];
    if (domain[2] == 1) l.views[i].stride[2] = 1;
  }
  for (int k = 0; k < 3; ++k) l.outStride[k] = store.stride[k];
  l.outStride[2] = 1;
  l.body = g.body;
  l.ctaThreads = static_cast<int>(optionalField(d.ctaThreadsField, tiling));
  l.unroll = static_cast<int>(optionalField(d.unrollField, tiling));
  l.gridBlocks = args.blockDim;
  // the innermost of the outer dims goes to the kernel library (it takes one as the grid's second dimension where
  // the group allows, and walks it itself where not); the others are walked here
  if (!outer.empty()) {
    l.outerCount = outer.back();
    for (size_t i = 0; i < loads.size(); ++i) l.viewOuterStride[i] = outerStride[i].back();
    l.outOuterStride = outerStride[loads.size()].back();
    outerCount /= outer.back();
    outer.pop_back();
    for (auto &strides : outerStride) strides.pop_back();
  }
  std::vector<int64_t> index(outer.size(), 0);
  for (int64_t launch = 0; launch < outerCount; ++launch) {
    auto shifted = [&](size_t view, const ResolvedView &v) {
      int64_t elems = 0;
      for (size_t j = 0; j < outer.size(); ++j) elems += index[j] * outerStride[view][j];
      return static_cast<char *>(argAt(args, v)) + elems * v.elemBytes;
    };
    for (size_t i = 0; i < loads.size(); ++i) l.views[i].base = shifted(i, loads[i]);
    l.outBase = shifted(loads.size(), store);
    int n = 0;
    Status s = cudaStatus(kernels::launchElementwise(l, args.stream, &n), "elementwise launch");
    info.kernelsLaunched += n;
    if (!s) return s;
    for (int j = static_cast<int>(outer.size()) - 1; j >= 0; --j) {
      if (++index[j] < outer[j]) break;
      index[j] = 0;
    }
  }
  return Status::success();
}

// Resolves a row-reduction group against concrete sizes and pointers: everything launchRowReduce needs.
Status buildRowReduceLaunch(const LaunchDescriptor &d, const GroupSpec &g, const std::map<std::string, int64_t> &tiling,
                            const LaunchArgs &args, kernels::RowReduceLaunch &l) {
  bool ok;
  const int et = toElemType(d.dtype, ok);
  if (!ok) return Status::error("row reductions compute in f32, f16 or bf16");
  std::vector<int64_t> domain;
  if (Status s = evalDims(g.domain, tiling, domain); !s) return s;
  if (domain.size() < 2) return Status::error("row reduction needs a [rows..., cols] domain");
  if (Status s = applyRowRange(domain, args); !s) return s;
  std::vector<ResolvedView> loads(g.loads.size());
  ResolvedView store;
  for (size_t i = 0; i < g.loads.size(); ++i)
    if (Status s = resolveView(g.loads[i], domain, tiling, args, "load", loads[i]); !s) return s;
  if (Status s = resolveView(g.store, domain, tiling, args, "store", store); !s) return s;
  if (store.stride.back() != 0) return Status::error("the reduced dim must not index the output");
  std::vector<ResolvedView *> all;
  for (auto &v : loads) all.push_back(&v);
  all.push_back(&store);
  // keep the reduced (last) dim apart: collapse only the leading dims
  const int64_t cols = domain.back();
  std::vector<int64_t> outer(domain.begin(), domain.end() - 1);
  std::vector<int64_t> colStride;
  for (auto *v : all) { colStride.push_back(v->stride.back()); v->stride.pop_back(); }
  collapseDomain(outer, all);
  if (outer.size() != 1) return Status::error("row reduction: leading dims do not collapse to one row dim");
  if (store.stride[0] != 1 && outer[0] != 1) return Status::error("row reduction: output rows must be contiguous");

  l = kernels::RowReduceLaunch();
  l.elemType = et;
  l.rows = outer[0];
  l.cols = cols;
  l.numViews = static_cast<int>(loads.size());
  for (size_t i = 0; i < loads.size(); ++i) {
    l.views[i].base = argAt(args, loads[i]);
    l.views[i].rowStride = loads[i].stride[0];
    l.views[i].colStride = colStride[i];
  }
  l.out = argAt(args, store);
  l.body = g.body;
  l.ctaThreads = static_cast<int>(optionalField(d.ctaThreadsField, tiling));
  l.teamLanes = static_cast<int>(optionalField(d.teamLanesField, tiling));
  l.streamStages = static_cast<int>(optionalField(d.streamStagesField, tiling));
  l.streamChunkBytes = static_cast<int>(optionalField(d.streamChunkField, tiling));
  if (!d.bulkCopyField.empty()) {
    auto it = tiling.find(d.bulkCopyField);
    if (it != tiling.end() && it->second == 0) l.forcePlainLoads = 1;
  }
  int split = static_cast<int>(optionalField(d.splitColsField, tiling));
  if (split <= 0) split = kernels::chooseRowReduceSplit(l.rows, l.cols, kernels::deviceSmCount(args.device));
  if (args.exchange) {
    if (args.rowEnd >= 0) return Status::error("row reduction: an exchange of partial sums does not take a row range");
    if (l.rows > args.exchange->slotStride)
      return Status::error("row reduction: " + std::to_string(l.rows) + " rows exceed the exchange's max_rows of " +
                           std::to_string(args.exchange->slotStride));
    l.exchange = args.exchange;
    split = 1;  // the partial sums of the exchange take the place of column slices
  }
  l.splitCols = split;
  if (split > 1) {
    const size_t need = kWorkspaceStatusBytes + kernels::rowReduceWorkspaceBytes(l.rows, split);
    if (!args.workspace || args.workspaceBytes < need)
      return Status::error("row reduction split into " + std::to_string(split) + " column slices needs " +
                           std::to_string(need) + " workspace bytes, " + std::to_string(args.workspaceBytes) + " given");
    l.workspace = static_cast<char *>(args.workspace) + kWorkspaceStatusBytes;
    l.workspaceBytes = args.workspaceBytes - kWorkspaceStatusBytes;
  }
  // wait time-outs of the staged kernel go to this launch's own status block (not to a word shared by the device)
  if (args.workspace && args.workspaceBytes >= kWorkspaceStatusBytes && !args.exchange)
    l.status = reinterpret_cast<unsigned int *>(static_cast<char *>(args.workspace) + kWorkspaceReduceStatusOffset);
  l.gridBlocks = args.blockDim;
  return Status::success();
}

Status launchRowReduceGroup(const LaunchDescriptor &d, const GroupSpec &g, const std::map<std::string, int64_t> &tiling,
                            const LaunchArgs &args, LaunchInfo &info) {
  kernels::RowReduceLaunch l;
  if (Status s = buildRowReduceLaunch(d, g, tiling, args, l); !s) return s;
  int n = 0;
  Status s = cudaStatus(kernels::launchRowReduce(l, args.stream, &n), "row-reduce launch");
  info.kernelsLaunched += n;
  if (l.status) info.usesStatusBlock = true;
  return s;
}

Status buildGatherLaunch(const LaunchDescriptor &d, const GroupSpec &g, const std::map<std::string, int64_t> &tiling,
                         const LaunchArgs &args, kernels::GatherLaunch &l, bool &usesStatusBlock) {
  bool ok;
  const int et = toElemType(d.dtype, ok);
  if (!ok) return Status::error("gather groups compute in f32, f16 or bf16");
  std::vector<int64_t> domain;
  if (Status s = evalDims(g.domain, tiling, domain); !s) return s;
  int64_t fullRows = 0;
  if (Status s = applyRowRange(domain, args, &fullRows); !s) return s;
  const int64_t rowShift = args.rowEnd >= 0 ? args.rowBegin : 0;
  // table: a plain 2-D argument
  const ViewSpec &tv = g.loads[0];
  std::vector<int64_t> tshape;
  if (Status s = evalDims(tv.shape, tiling, tshape); !s) return s;
  if (tshape.size() != 2) return Status::error("gather table must be 2-D");
  if (args.argBytes[tv.arg] != static_cast<size_t>(tshape[0] * tshape[1]) * dtypeBytes(tv.dtype))
    return Status::error("gather table: argument " + std::to_string(tv.arg) + " byte size does not match the tiling dims");
  if (tv.dtype != d.dtype) return Status::error("gather table differs from the group element type");
  std::vector<int64_t> ishape;
  if (Status s = evalDims(g.indices.shape, tiling, ishape); !s) return s;
  const int64_t wantIdx = g.gatherAxis == 0 ? fullRows : domain[1];
  if (ishape.size() != 1 || ishape[0] != wantIdx) return Status::error("gather indices: expected a vector of " + std::to_string(wantIdx));
  if (args.argBytes[g.indices.arg] != static_cast<size_t>(wantIdx) * dtypeBytes(g.indices.dtype))
    return Status::error("gather indices: argument byte size does not match");
  if (g.gatherAxis == 0 && tshape[1] != domain[1]) return Status::error("row gather: table width differs from the output width");
  if (g.gatherAxis == 1 && tshape[0] != fullRows) return Status::error("column gather: table rows differ from the output rows");

  std::vector<ResolvedView> loads(g.loads.size());
  ResolvedView store;
  for (size_t i = 1; i < g.loads.size(); ++i) {
    if (g.loads[i].dtype != d.dtype) return Status::error("load " + std::to_string(i) + " differs from the group element type");
    if (Status s = resolveView(g.loads[i], domain, tiling, args, "load", loads[i]); !s) return s;
  }
  if (Status s = resolveView(g.store, domain, tiling, args, "store", store); !s) return s;
  if (store.stride[1] != 1 && domain[1] != 1) return Status::error("gather: output must be contiguous along the inner dim");

  l = kernels::GatherLaunch();
  l.elemType = et;
  l.axis = g.gatherAxis;
  l.indexType = g.indices.dtype == DType::I64 ? kernels::kI64 : kernels::kI32;
  l.rows = domain[0];
  l.cols = domain[1];
  l.table = args.argPtrs[tv.arg];
  if (g.gatherAxis == 1)  // output row i reads table row i: a row range shifts the table too
    l.table = static_cast<const char *>(l.table) + static_cast<size_t>(rowShift * tshape[1]) * dtypeBytes(tv.dtype);
  l.tableRows = tshape[0];
  l.tableCols = tshape[1];
  l.tableRowStride = tshape[1];
  if (!args.tableShards.empty()) {
    if (g.gatherAxis != 0) return Status::error("a sharded table needs a row gather");
    if (args.tableShards.size() > static_cast<size_t>(kernels::kMaxTableShards))
      return Status::error("a table takes at most " + std::to_string(kernels::kMaxTableShards) + " shards");
    if (args.rowsPerShard <= 0 || args.rowsPerShard * static_cast<int64_t>(args.tableShards.size()) < tshape[0])
      return Status::error("table shards: " + std::to_string(args.tableShards.size()) + " shards of " + std::to_string(args.rowsPerShard) +
                           " rows do not cover the table's " + std::to_string(tshape[0]) + " rows");
    if (tshape[0] >= (1ll << 32)) return Status::error("a sharded table has fewer than 2^32 rows");
    l.numShards = static_cast<int>(args.tableShards.size());
    for (int sh = 0; sh < l.numShards; ++sh) {
      if (!args.tableShards[sh]) return Status::error("table shard " + std::to_string(sh) + " is null");
      l.tableShards[sh] = args.tableShards[sh];
    }
    l.rowsPerShard = args.rowsPerShard;
    l.table = nullptr;
  }
  l.indices = args.argPtrs[g.indices.arg];
  if (g.gatherAxis == 0)
    l.indices = static_cast<const char *>(l.indices) + static_cast<size_t>(rowShift) * dtypeBytes(g.indices.dtype);
  l.numViews = static_cast<int>(g.loads.size());
  for (size_t i = 1; i < loads.size(); ++i) {
    l.views[i].base = argAt(args, loads[i]);
    l.views[i].rowStride = loads[i].stride[0];
    l.views[i].colStride = loads[i].stride[1];
  }
  l.out = argAt(args, store);
  l.outRowStride = store.stride[0];
  l.body = g.body;
  if (args.workspace && args.workspaceBytes >= kWorkspaceStatusBytes) {
    l.status = static_cast<unsigned long long *>(args.workspace);
    usesStatusBlock = true;
  }
  l.ctaThreads = static_cast<int>(optionalField(d.ctaThreadsField, tiling));
  l.unroll = static_cast<int>(optionalField(d.unrollField, tiling));
  l.gridBlocks = args.blockDim;
  if (!d.bulkCopyField.empty()) {
    auto it = tiling.find(d.bulkCopyField);
    if (it != tiling.end() && it->second == 1) l.stagedCopies = 1;
  }
  l.streamStages = static_cast<int>(optionalField(d.streamStagesField, tiling));
  l.streamRows = static_cast<int>(optionalField(d.streamRowsField, tiling));
  l.streamWarps = static_cast<int>(optionalField(d.streamWarpsField, tiling));
  return Status::success();
}

Status launchGatherGroup(const LaunchDescriptor &d, const GroupSpec &g, const std::map<std::string, int64_t> &tiling,
                         const LaunchArgs &args, LaunchInfo &info) {
  kernels::GatherLaunch l;
  bool usesStatus = false;
  if (Status s = buildGatherLaunch(d, g, tiling, args, l, usesStatus); !s) return s;
  if (usesStatus) info.usesStatusBlock = true;
  int n = 0;
  Status s = cudaStatus(kernels::launchGather(l, args.stream, &n), "gather launch");
  info.kernelsLaunched += n;
  return s;
}

Status launchTransposeGroup(const LaunchDescriptor &d, const GroupSpec &g, const std::map<std::string, int64_t> &tiling,
                            const LaunchArgs &args, LaunchInfo &info) {
  // domain = output shape [C, R]; loads[0] is the [R, C] input read as (d1, d0)
  std::vector<int64_t> domain;
  if (Status s = evalDims(g.domain, tiling, domain); !s) return s;
  if (args.rowEnd >= 0) return Status::error("transpose groups do not take a row range");
  if (domain.size() != 2 || g.loads.size() != 1 || g.body.numOps != 0)
    return Status::error("transpose groups are a bare 2-D permutation of one input");
  ResolvedView in, store;
  if (Status s = resolveView(g.loads[0], domain, tiling, args, "load", in); !s) return s;
  if (Status s = resolveView(g.store, domain, tiling, args, "store", store); !s) return s;
  if (in.stride[0] != 1 || store.stride[1] != 1) return Status::error("transpose: expected the input to be read column-wise");
  kernels::TransposeLaunch l = {};
  l.elemBytes = static_cast<int>(dtypeBytes(d.dtype));
  l.rows = domain[1];
  l.cols = domain[0];
  l.in = argAt(args, in);
  l.inRowStride = in.stride[1];
  l.out = argAt(args, store);
  l.outRowStride = store.stride[0];
  l.warpRows = static_cast<int>(optionalField(d.warpRowsField, tiling));
  l.ctasPerSm = static_cast<int>(optionalField(d.ctasPerSmField, tiling));
  l.forceTileKernel = optionalField(d.tileKernelField, tiling) != 0;
  l.diagonalOrder = static_cast<int>(optionalField(d.tileOrderField, tiling));  // 0, 1 or 2
  l.variant = static_cast<int>(optionalField(d.variantField, tiling));
  if (args.workspace && args.workspaceBytes >= kWorkspaceStatusBytes) {
    l.status = reinterpret_cast<unsigned int *>(static_cast<char *>(args.workspace) + kWorkspaceTransposeStatusOffset);
    info.usesStatusBlock = true;
  }
  int n = 0;
  Status s = cudaStatus(kernels::launchTranspose(l, args.stream, &n), "transpose launch");
  info.kernelsLaunched += n;
  return s;
}

Status launchMatmulDescriptor(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args,
                              LaunchInfo &info) {
  const MatmulSpec &m = d.matmul;
  int64_t M, N, K;
  if (Status s = evalDim(m.m, tiling, M); !s) return s;
  if (Status s = evalDim(m.n, tiling, N); !s) return s;
  if (Status s = evalDim(m.k, tiling, K); !s) return s;
  bool ok1, ok2, ok3;
  kernels::MatmulLaunch l = {};
  l.inType = toElemType(m.inType, ok1);
  l.outType = toElemType(m.outType, ok2);
  l.biasType = toElemType(m.biasType, ok3);
  if (!ok1 || !ok2 || !ok3 || m.inType == DType::F32) return Status::error("matmul: inputs are f16 or bf16; bias/out f32, f16 or bf16");
  auto check = [&](int arg, int64_t elems, DType t, const char *name) -> Status {
    const size_t want = static_cast<size_t>(elems) * dtypeBytes(t);
    if (args.argBytes[arg] != want)
      return Status::error(std::string("[cuda:bindings] matmul ") + name + ": argument " + std::to_string(arg) + " is " +
                           std::to_string(args.argBytes[arg]) + " bytes, the tiling dims imply " + std::to_string(want));
    return Status::success();
  };
  if (Status s = check(m.aArg, M * K, m.inType, "A"); !s) return s;
  if (Status s = check(m.bArg, K * N, m.inType, "B"); !s) return s;
  if (m.biasArg >= 0)
    if (Status s = check(m.biasArg, N, m.biasType, "bias"); !s) return s;
  if (Status s = check(m.outArg, M * N, m.outType, "out"); !s) return s;
  int64_t r0 = 0, r1 = M;
  if (args.rowEnd >= 0) {
    if (args.rowBegin < 0 || args.rowBegin > args.rowEnd || args.rowEnd > M) return Status::error("row range outside M");
    r0 = args.rowBegin;
    r1 = args.rowEnd;
  }
  l.M = r1 - r0; l.N = N; l.K = K;
  l.A = static_cast<const char *>(args.argPtrs[m.aArg]) + static_cast<size_t>(r0 * K) * dtypeBytes(m.inType);
  l.B = args.argPtrs[m.bArg];
  l.bias = m.biasArg >= 0 ? args.argPtrs[m.biasArg] : nullptr;
  l.out = static_cast<char *>(args.argPtrs[m.outArg]) + static_cast<size_t>(r0 * N) * dtypeBytes(m.outType);
  l.epilogue = m.epilogue;
  l.alpha = static_cast<float>(m.alpha);
  l.bTransposed = m.transposeB ? 1 : 0;
  l.gridBlocks = args.blockDim;
  l.stages = static_cast<int>(optionalField(d.stagesField, tiling));
  if (args.workspace && args.workspaceBytes >= kWorkspaceStatusBytes) {
    l.status = reinterpret_cast<unsigned int *>(static_cast<char *>(args.workspace) + kWorkspaceMatmulStatusOffset);
    info.usesStatusBlock = true;
  }
  int n = 0;
  char text[256] = {0};
  kernels::MatmulPlan plan;
  l.planOut = &plan;
  const int code = kernels::launchMatmul(l, args.stream, &n, text);
  info.kernelsLaunched += n;
  if (code != 0) return Status::error(text[0] ? std::string(text) : std::string("matmul launch: ") + kernels::cudaErrorText(code));
  if (n > 0) info.plan = kernels::describeMatmulPlan(plan);
  return Status::success();
}

} // namespace

Status requiredWorkspaceBytes(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, int device, size_t &bytes) {
  bytes = kWorkspaceStatusBytes;
  if (d.kernelClass != KernelClass::RowReduce) return Status::success();
  for (const auto &g : d.groups) {
    std::vector<int64_t> domain;
    if (Status s = evalDims(g.domain, tiling, domain); !s) return s;
    if (domain.size() < 2) continue;
    int64_t rows = 1;
    for (size_t i = 0; i + 1 < domain.size(); ++i) rows *= domain[i];
    int split = static_cast<int>(optionalField(d.splitColsField, tiling));
    if (split <= 0) split = kernels::chooseRowReduceSplit(rows, domain.back(), kernels::deviceSmCount(device));
    bytes = std::max(bytes, kWorkspaceStatusBytes + kernels::rowReduceWorkspaceBytes(rows, split));
  }
  return Status::success();
}

Status launchDescriptor(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args,
                        LaunchInfo &info) {
  info = LaunchInfo();
  const size_t numArgs = static_cast<size_t>(d.numInputs + d.numOutputs);
  if (args.argPtrs.size() != numArgs || args.argBytes.size() != numArgs)
    return Status::error("kernel '" + d.kernel + "' takes " + std::to_string(d.numInputs) + " inputs and " +
                         std::to_string(d.numOutputs) + " outputs");
  if (args.exchange && (d.kernelClass != KernelClass::RowReduce || d.groups.size() != 1))
    return Status::error("only a single row-reduction group exchanges partial sums between GPUs");
  if (!args.tableShards.empty() && (d.kernelClass != KernelClass::Gather || d.groups.size() != 1))
    return Status::error("only a single gather group takes a sharded table");
  if (d.kernelClass == KernelClass::Matmul) return launchMatmulDescriptor(d, tiling, args, info);
  for (const auto &g : d.groups) {
    Status s;
    switch (d.kernelClass) {
    case KernelClass::Elementwise: s = launchElementwiseGroup(d, g, tiling, args, info); break;
    case KernelClass::RowReduce: s = launchRowReduceGroup(d, g, tiling, args, info); break;
    case KernelClass::Gather: s = launchGatherGroup(d, g, tiling, args, info); break;
    case KernelClass::Transpose: s = launchTransposeGroup(d, g, tiling, args, info); break;
    default: s = Status::error("unsupported kernel class"); break;
    }
    if (!s) return s;
  }
  return Status::success();
}


// ---- generated kernels ---------------------------------------------------------------------------------------------
bool generatedLaunchApplies(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args) {
  if (args.exchange || !args.tableShards.empty()) return false;
  if (!args.workspace || args.workspaceBytes < kWorkspaceStatusBytes) return false;  // status words live there
  switch (d.kernelClass) {
  case KernelClass::Elementwise: {
    const int64_t unroll = optionalField(d.unrollField, tiling);
    return unroll == 0 || unroll == 2;  // the generated loop keeps two vectors per thread in flight
  }
  case KernelClass::RowReduce: return true;
  case KernelClass::Gather: {
    if (d.groups.size() != 1 || d.groups[0].gatherAxis != 0) return false;
    if (!d.bulkCopyField.empty()) {
      auto it = tiling.find(d.bulkCopyField);
      if (it != tiling.end() && it->second == 1) return false;  // the staged-copy experiment is a prebuilt kernel
    }
    const int64_t unroll = optionalField(d.unrollField, tiling);
    return unroll == 0 || unroll == 1 || unroll == 2;
  }
  default: return false;
  }
}

namespace {

int clampThreads(int64_t requested) {
  int threads = requested > 0 ? static_cast<int>(std::min<int64_t>(requested, 512)) : 128;
  return std::max(32, std::min(512, (threads / 32) * 32));
}

// Kernel arguments in the reference's order: inputs..., outputs..., workspace, TilingData (all-int64: the
// descriptor's fields, then the row window and the six plan words).
struct GeneratedArgs {
  std::vector<void *> pointers;
  void *workspace = nullptr;
  std::vector<int64_t> words;
  std::vector<void *> params;

  GeneratedArgs(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args) {
    pointers = args.argPtrs;
    workspace = args.workspace;
    for (const TilingField &f : d.tiling) {
      auto it = tiling.find(f.name);
      words.push_back(it == tiling.end() ? 0 : it->second);
    }
    const size_t hidden = words.size();
    words.resize(hidden + 8, 0);
    words[hidden + 0] = args.rowEnd >= 0 ? args.rowBegin : 0;
    words[hidden + 1] = args.rowEnd >= 0 ? args.rowEnd : -1;
    planBase_ = hidden + 2;
  }
  void setPlan(int index, int64_t value) { words[planBase_ + static_cast<size_t>(index)] = value; }
  void **finish() {
    params.clear();
    for (void *&p : pointers) params.push_back(&p);
    params.push_back(&workspace);
    params.push_back(words.data());
    return params.data();
  }

private:
  size_t planBase_ = 0;
};

} // namespace

Status launchGenerated(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling, const LaunchArgs &args,
                       GeneratedBinding &binding, LaunchInfo &info) {
  info = LaunchInfo();
  info.generated = true;
  const size_t numArgs = static_cast<size_t>(d.numInputs + d.numOutputs);
  if (args.argPtrs.size() != numArgs || args.argBytes.size() != numArgs)
    return Status::error("kernel '" + d.kernel + "' takes " + std::to_string(d.numInputs) + " inputs and " +
                         std::to_string(d.numOutputs) + " outputs");
  if (!binding.module || !binding.mainFn) return Status::error("kernel '" + d.kernel + "' has no generated code loaded");
  GeneratedArgs ga(d, tiling, args);

  if (d.kernelClass == KernelClass::Elementwise) {
    // (a kernel with the register-block loop of transposed operands is compiled for CTAs of 256 threads)
    const int threads = binding.ctasOf256Threads ? 256 : clampThreads(optionalField(d.ctaThreadsField, tiling));
    int64_t tiles = 1;
    int64_t totalElems = 0;
    for (const GroupSpec &g : d.groups) {
      int et = 0;
      std::vector<int64_t> domain;
      std::vector<ResolvedView> loads;
      ResolvedView store;
      if (Status s = resolveElementwiseGroup(d, g, tiling, args, et, domain, loads, store); !s) return s;
      int64_t elems = 1;
      for (int64_t e : domain) elems *= e;
      // A group that reads an operand through a transposed view has the register-block loop in its kernel: one CTA
      // per tile of 2 x 4 warps x 4 x 8 blocks when everything is aligned for 16-byte pieces (the kernel tests the
      // same, on its own view of the dims), else one element per thread and step.  Both loops walk their tiles with a
      // grid stride, so a grid that guesses the other loop costs time, not results.
      int64_t transposedTiles = 0;
      if (binding.ctasOf256Threads) {
        std::vector<ResolvedView> copies = loads;
        ResolvedView storeCopy = store;
        std::vector<int64_t> dom = domain;
        std::vector<ResolvedView *> all;
        for (auto &v : copies) all.push_back(&v);
        all.push_back(&storeCopy);
        collapseDomain(dom, all);
        if (dom.size() <= 3 && !dom.empty()) {
          while (dom.size() < 3) {
            dom.insert(dom.begin(), 1);
            for (auto *v : all) v->stride.insert(v->stride.begin(), 0);
          }
          const int64_t e = 16 / static_cast<int64_t>(dtypeBytes(d.dtype));
          auto aligned = [&](const ResolvedView &v, int64_t sa, int64_t sb) {
            return (reinterpret_cast<uintptr_t>(argAt(args, v)) & 15u) == 0 && sa % e == 0 && sb % e == 0;
          };
          bool transposed = false, blocks = aligned(storeCopy, storeCopy.stride[0], storeCopy.stride[1]);
          for (const ResolvedView &v : copies) {
            if (v.stride[2] == 1) blocks = blocks && aligned(v, v.stride[0], v.stride[1]);
            else if (v.stride[2] != 0 && v.stride[1] == 1 && dom[2] != 1) { transposed = true; blocks = blocks && aligned(v, v.stride[0], v.stride[2]); }
            else if (v.stride[2] != 0) blocks = false;
          }
          if (transposed)
            transposedTiles = blocks ? dom[0] * ((dom[2] + 32 * e - 1) / (32 * e)) * ((dom[1] + 8 * e - 1) / (8 * e))
                                     : (elems + threads * 2 - 1) / (threads * 2);
        }
      }
      // the kernel counts 16-byte vectors (or elements, when something is unaligned) in 32 bits
      if (elems >= (1ll << 32) - (1 << 20)) return Status::error("[generated:unsupported] more than 2^32 elements in one group");
      totalElems += elems;
      const int64_t vecs = (elems + (16 / static_cast<int64_t>(dtypeBytes(d.dtype))) - 1) / (16 / static_cast<int64_t>(dtypeBytes(d.dtype)));
      tiles = std::max(tiles, transposedTiles > 0 ? transposedTiles : (vecs + threads * 2 - 1) / (threads * 2));
    }
    if (totalElems == 0) return Status::success();
    int64_t grid = args.blockDim > 0 ? std::min<int64_t>(args.blockDim, tiles) : tiles;
    grid = std::max<int64_t>(1, std::min<int64_t>(grid, 0x7fffffff));
    if (Status s = launchDeviceFunction(binding.mainFn, static_cast<unsigned int>(grid), static_cast<unsigned int>(threads), 0, args.stream, ga.finish(), binding.waitsForDependencies); !s)
      return s;
    info.kernelsLaunched = 1;
    return Status::success();
  }

  if (d.kernelClass == KernelClass::RowReduce) {
    if (d.groups.size() != 1) return Status::error("one group per row-reduction kernel");
    kernels::RowReduceLaunch l;
    if (Status s = buildRowReduceLaunch(d, d.groups[0], tiling, args, l); !s) return s;
    if (l.rows == 0) return Status::success();
    kernels::RowReducePlan plan;
    if (const int rc = kernels::planRowReduce(l, kernels::deviceSmCount(args.device), plan); rc != 0)
      return cudaStatus(rc, "row-reduce launch");
    info.usesStatusBlock = true;
    if (plan.staged && binding.stagedFn) {
      ga.setPlan(0, plan.streamStages);
      ga.setPlan(1, plan.streamChunkBytes);
      if (Status s = binding.module->reserveDynamicSharedMemory(binding.stagedFn, static_cast<int>(plan.smemBytes)); !s) return s;
      if (Status s = launchDeviceFunction(binding.stagedFn, static_cast<unsigned int>(plan.grid), static_cast<unsigned int>(plan.threads),
                                          plan.smemBytes, args.stream, ga.finish(), binding.waitsForDependencies); !s)
        return s;
      info.kernelsLaunched = 1;
      return Status::success();
    }
    if (plan.staged) {  // no staged entry in this module: plan again for plain loads
      l.forcePlainLoads = 1;
      if (const int rc = kernels::planRowReduce(l, kernels::deviceSmCount(args.device), plan); rc != 0)
        return cudaStatus(rc, "row-reduce launch");
    }
    ga.setPlan(0, plan.vector ? 1 : 0);
    ga.setPlan(1, plan.slices);
    ga.setPlan(2, plan.vecPerSlice);
    ga.setPlan(3, plan.lanes);
    if (Status s = launchDeviceFunction(binding.mainFn, static_cast<unsigned int>(plan.grid), static_cast<unsigned int>(plan.threads), 0,
                                        args.stream, ga.finish(), binding.waitsForDependencies); !s)
      return s;
    info.kernelsLaunched = 1;
    if (plan.slices > 1) {
      if (!binding.finalizeFn) return Status::error("kernel '" + d.kernel + "' has no finalize entry for its column slices");
      if (Status s = launchDeviceFunction(binding.finalizeFn, static_cast<unsigned int>(plan.finalizeGrid),
                                          static_cast<unsigned int>(plan.finalizeThreads), 0, args.stream, ga.finish(), binding.waitsForDependencies); !s)
        return s;
      info.kernelsLaunched = 2;
    }
    return Status::success();
  }

  if (d.kernelClass == KernelClass::Gather) {
    if (d.groups.size() != 1) return Status::error("one group per gather kernel");
    kernels::GatherLaunch l;
    bool usesStatus = false;
    if (Status s = buildGatherLaunch(d, d.groups[0], tiling, args, l, usesStatus); !s) return s;
    info.usesStatusBlock = true;
    if (l.rows == 0 || l.cols == 0) return Status::success();
    const int eb = kernels::elemBytes(l.elemType);
    const int64_t vecPerRow = (l.cols + 16 / eb - 1) / (16 / eb);
    if (l.rows * l.cols >= (1ll << 32) - (1 << 20)) return Status::error("[generated:unsupported] more than 2^32 elements in one group");
    const int threads = clampThreads(l.ctaThreads);
    const int inFlight = l.unroll == 2 ? 2 : 1;
    ga.setPlan(0, inFlight);
    auto divisionWord = [](int64_t divisor) {  // kernels::makeFastDiv, packed as magic | shift << 32
      const unsigned int d = static_cast<unsigned int>(std::max<int64_t>(1, divisor));
      unsigned int shift = 0;
      while ((1ull << shift) < d) ++shift;
      const unsigned int magic = static_cast<unsigned int>(((1ull << 32) * ((1ull << shift) - d)) / d + 1);
      return static_cast<int64_t>(static_cast<uint64_t>(magic) | (static_cast<uint64_t>(shift) << 32));
    };
    ga.setPlan(1, divisionWord(l.cols / (16 / eb)));
    ga.setPlan(2, divisionWord(l.cols));
    const int64_t tileVecs = static_cast<int64_t>(threads) * inFlight;
    const int64_t tiles = (l.rows * vecPerRow + tileVecs - 1) / tileVecs;
    // A generated kernel works its views and strides out of TilingData at the start of every CTA, which a CTA of
    // one tile (one or two vectors per thread) does not pay back: the grid stops at four times the threads an SM can
    // hold and the CTAs walk the tiles (measured on 262 144 x 256 bf16: 0.89 of the copy rate with one tile per CTA,
    // 0.98-0.99 so).
    const int64_t resident = static_cast<int64_t>(kernels::deviceSmCount(args.device)) * (8192 / threads);
    int64_t grid = args.blockDim > 0 ? std::min<int64_t>(args.blockDim, tiles) : std::min(tiles, resident);
    grid = std::max<int64_t>(1, std::min<int64_t>(grid, 0x7fffffff));
    void *fn = inFlight == 1 && binding.singleVectorFn ? binding.singleVectorFn : binding.mainFn;
    if (Status s = launchDeviceFunction(fn, static_cast<unsigned int>(grid), static_cast<unsigned int>(threads), 0, args.stream, ga.finish(), binding.waitsForDependencies); !s)
      return s;
    info.kernelsLaunched = 1;
    return Status::success();
  }
  return Status::error("kernel class has no generated code");
}

} // namespace afir

namespace afir {
namespace {

// Marks argument `arg` as row-sliced with `bytes` per leading-dim row; conflicting uses make chunking impossible.
bool noteSlice(std::vector<size_t> &rowBytes, std::vector<char> &seen, int arg, size_t bytes) {
  if (arg < 0 || arg >= static_cast<int>(rowBytes.size())) return false;
  if (seen[arg] && rowBytes[arg] != bytes) return false;
  seen[arg] = 1;
  rowBytes[arg] = bytes;
  return true;
}

// A view is chunkable when the leading iteration dim does not index it at all (whole argument needed by
// every chunk), or indexes its outermost tensor dim starting at offset 0 (rows are contiguous byte ranges).
bool classifyView(const ViewSpec &v, const std::map<std::string, int64_t> &tiling, std::vector<size_t> &rowBytes,
                  std::vector<char> &seen) {
  int mapped = -1;
  for (size_t t = 0; t < v.map.size(); ++t)
    if (v.map[t] == 0) {
      if (mapped >= 0) return false;
      mapped = static_cast<int>(t);
    }
  if (mapped < 0) return noteSlice(rowBytes, seen, v.arg, 0);
  if (mapped != 0) return false;
  if (!v.offset.empty()) {
    int64_t off = 0;
    if (!evalDim(v.offset[0], tiling, off) || off != 0) return false;
  }
  std::vector<int64_t> shape;
  if (!evalDims(v.shape, tiling, shape)) return false;
  size_t bytes = dtypeBytes(v.dtype);
  for (size_t t = 1; t < shape.size(); ++t) bytes *= static_cast<size_t>(shape[t]);
  if (bytes == 0) return false;
  return noteSlice(rowBytes, seen, v.arg, bytes);
}

} // namespace

Status planRowPipeline(const LaunchDescriptor &d, const std::map<std::string, int64_t> &tiling,
                       const std::vector<size_t> &argBytes, RowPipelinePlan &plan) {
  plan = RowPipelinePlan();
  plan.rowBytes.assign(argBytes.size(), 0);
  std::vector<char> seen(argBytes.size(), 0);
  if (d.kernelClass == KernelClass::Matmul) {
    const MatmulSpec &m = d.matmul;
    int64_t M, N, K;
    if (Status s = evalDim(m.m, tiling, M); !s) return s;
    if (Status s = evalDim(m.n, tiling, N); !s) return s;
    if (Status s = evalDim(m.k, tiling, K); !s) return s;
    plan.rows = M;
    plan.possible = noteSlice(plan.rowBytes, seen, m.aArg, static_cast<size_t>(K) * dtypeBytes(m.inType)) &&
                    noteSlice(plan.rowBytes, seen, m.outArg, static_cast<size_t>(N) * dtypeBytes(m.outType)) && K > 0 && N > 0;
    return Status::success();
  }
  if (d.kernelClass == KernelClass::Transpose || d.groups.size() != 1) return Status::success();
  const GroupSpec &g = d.groups[0];
  std::vector<int64_t> domain;
  if (Status s = evalDims(g.domain, tiling, domain); !s) return s;
  if (domain.empty()) return Status::success();
  plan.rows = domain[0];
  bool ok = true;
  const bool gather = d.kernelClass == KernelClass::Gather;
  for (size_t i = 0; i < g.loads.size() && ok; ++i) {
    if (gather && i == 0) {
      // the table: whole for a row gather; row i of the output reads row i of it for a column gather
      std::vector<int64_t> tshape;
      if (!evalDims(g.loads[0].shape, tiling, tshape) || tshape.size() != 2) { ok = false; break; }
      ok = noteSlice(plan.rowBytes, seen, g.loads[0].arg,
                     g.gatherAxis == 1 ? static_cast<size_t>(tshape[1]) * dtypeBytes(g.loads[0].dtype) : 0);
      continue;
    }
    ok = classifyView(g.loads[i], tiling, plan.rowBytes, seen);
  }
  if (ok && gather)
    ok = noteSlice(plan.rowBytes, seen, g.indices.arg, g.gatherAxis == 0 ? dtypeBytes(g.indices.dtype) : 0);
  if (ok) ok = classifyView(g.store, tiling, plan.rowBytes, seen) && plan.rowBytes[g.store.arg] > 0;
  // every sliced argument must be exactly rows * rowBytes long
  for (size_t a = 0; a < argBytes.size() && ok; ++a)
    if (plan.rowBytes[a] && plan.rowBytes[a] * static_cast<size_t>(plan.rows) != argBytes[a]) ok = false;
  plan.possible = ok;
  return Status::success();
}

} // namespace afir
