// Conversion/AFIRToCUDA: classify one function (a fused group written as AFIR elementwise ops or as
// linalg-on-tensors) into a kernel class of the sm_100a library and build its launch descriptor and tiling
// space.  It plays the role of the reference's device lowering chain (LinalgToAscendC ... CannKernel,
// lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:244-1845) for this backend: elementwise producers are
// fused into their consumers symbolically (what --linalg-fuse-elementwise-ops achieves), gathers are detected
// by the five conditions of lib/Conversion/MarkStructuredOps/MarkStructuredOpsPass.cpp:54-139 and fused with
// their pre/post ops (lib/Conversion/FuseGatherElementwise/FuseGatherElementwisePass.cpp:61-303), matmul
// epilogues are matched as lib/Conversion/MarkStructuredOps/AnnotateMixMatmulSemanticsPass.cpp:171-242 does.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "common/json.h"
#include "front/mlir_text.h"

namespace afir {
namespace front {

struct GroupAnalysis {
  std::string kernelClass;   // elementwise | row_reduce | gather | matmul
  std::string kernelKind;    // vec | cube | mix   (the reference's ascendc.kernel_kind vocabulary)
  json::Value descriptor;    // afir-cuda-launch
  json::Value tilingSpace;   // tiling_space.json
  // per-op annotations found on the way: op index in the function -> (attribute, value text)
  std::map<size_t, std::vector<std::pair<std::string, std::string>>> opAttrs;
  // function-level attributes (kernel kind, matmul semantics)
  std::vector<std::pair<std::string, std::string>> funcAttrs;
};

Status analyzeFunction(const Module &module, const Func &func, GroupAnalysis &out);

} // namespace front
} // namespace afir
