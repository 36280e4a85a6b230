// --afir-shape-inference: refines the result types of afir elementwise ops from their operand types and carries
// the refined types to the ops that use them, to the return op and to the function's result types.  Restates the
// reference's pass (lib/Dialect/AFIR/Transforms/AFIRInferShapes.cpp:94-176) over its inference rule for
// broadcasting elementwise ops (lib/Dialect/AFIR/Ops/Basic/math.cpp:275-312) and its join of what the result type
// already says with what was inferred (include/Utils/AFIRShapeInferUtils.h:80-125).
#pragma once

#include <vector>

#include "front/mlir_text.h"

namespace afir {
namespace front {

// Trailing-aligned broadcast of operand shapes (-1 = dynamic).  The rank is the largest operand rank; at every
// position, from the last to the first and over the operands in order, an extent of 1 is skipped, the first other
// extent replaces a 1 or a dynamic entry, a later dynamic extent changes nothing, and two different static extents
// make the inference fail (false; `out` is then unspecified).
bool inferBroadcastShape(const std::vector<std::vector<int64_t>> &operands, std::vector<int64_t> &out);

// afir.concat (lib/Dialect/AFIR/Ops/Adv/concat.cpp:86-131): operands of one rank; along `axis` the static extents add up
// (one dynamic extent makes the sum dynamic), every other position takes the operands' common static extent and is
// dynamic as soon as one operand is dynamic there; operands that disagree, ranks that differ or an axis outside the
// rank make the inference fail.
bool inferConcatShape(const std::vector<std::vector<int64_t>> &operands, int64_t axis, std::vector<int64_t> &out);

// The afir reductions (sum, max, min, mean, prod, any, all; lib/Dialect/AFIR/Ops/Adv/reduce.cpp:72-91): the operand's
// shape with `axis` removed; an axis outside the rank makes the inference fail.
bool inferReducedShape(const std::vector<int64_t> &operand, int64_t axis, std::vector<int64_t> &out);

// What two descriptions of one shape agree on: a dynamic entry yields to a static one, equal entries stay; ranks
// or static extents that differ are a conflict (false).
bool joinShapes(const std::vector<int64_t> &current, const std::vector<int64_t> &inferred, std::vector<int64_t> &out);

// Runs the pass over every function of the module: updates the parsed types in place and records the text
// replacements printModule applies.  `refined` (optional) counts the op results whose type changed.  An op whose
// shapes do not broadcast, or whose declared result contradicts the inference, is left as it is, as in the reference.
void inferAfirShapes(Module &m, int *refined = nullptr);

} // namespace front
} // namespace afir
