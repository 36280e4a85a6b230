// Printing a fused group back as ONE linalg.generic: what the reference's --linalg-fuse-elementwise-ops leaves
// behind for an elementwise / broadcast / reduction chain (upstream MLIR's pass) and what its
// --fuse-gather-elementwise builds for a gather with pre- and post-ops
// (lib/Conversion/FuseGatherElementwise/FuseGatherElementwisePass.cpp:61-303: one gather generic whose body is
// pre-op -> tensor.extract -> post-ops, reading the index vector and the broadcast extras).  The group analysis
// already holds the fused body symbolically; this turns it into text and replaces the group's generics by it.
#pragma once

#include <string>

#include "front/group_analysis.h"

namespace afir {
namespace front {

// Rewrites `func` inside `module` (as replacements / erasures for printModule) so that its generics become one
// fused generic.  Returns false, with the reason in `why`, when the function is left as it is: a single generic
// already, a matmul, a bare transpose, or views that are slices of an argument (split / concat groups keep their
// tensor.extract_slice / insert_slice form).
bool fuseGenericsInPlace(Module &module, const Func &func, const GroupAnalysis &analysis, std::string &why);

} // namespace front
} // namespace afir
