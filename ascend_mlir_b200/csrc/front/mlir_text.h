// Self-contained reader for the textual MLIR subset the fused-group front end consumes (MLIR itself is not
// a dependency): module / func.func, affine_map aliases, tensor types with dynamic dims, arith.constant,
// tensor.{dim,empty,extract_slice,concat,extract}, linalg.{generic,matmul,fill,index,yield}, the arith ops
// fused bodies use, afir.{add,sub,mul,div,truediv,minimum,maximum,relu,leaky_relu,neg,abs,clip_by_value,concat,sum} (the other
// reductions parse and take part in shape inference only), return.  This is the input language of the reference's examples
// (examples/*/step0_input.mlir) and of its AFIR elementwise ops (include/Dialect/AFIR/Ops/Basic/math.td:60-121).
// Anything outside the subset is a parse error naming the op: nothing is skipped silently.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "common/status.h"

namespace afir {
namespace front {

struct Type {
  bool isTensor = false;
  std::vector<int64_t> dims;  // -1 = dynamic
  std::string elem;           // f16, bf16, f32, i32, i64, index, ...
  std::string str() const;
};

// Projected permutation with optional constant-0 results: result r is iteration dim results[r], or -1 for 0.
struct AffineMap {
  int numDims = 0;
  std::vector<int> results;
  std::string str() const;
};

// An index operand that is either a literal or an SSA value.
struct IndexOperand {
  bool literal = true;
  int64_t value = 0;
  std::string ssa;
};

struct Op {
  std::string name;                   // "linalg.generic", "arith.addf", ...
  std::vector<std::string> results;   // SSA names without '%'
  std::vector<std::string> operands;
  std::vector<Type> operandTypes;
  Type resultType;
  // arith.constant
  double constFloat = 0.0;
  int64_t constInt = 0;
  bool constIsFloat = false;
  // linalg.generic / matmul / fill
  std::vector<AffineMap> maps;
  std::vector<std::string> iterators;
  int numIns = 0;                     // operands[0..numIns) are ins, the rest outs
  std::string unit;                   // value of an ascendc.unit attribute on the op ("AiCore.Cube", "AiCore.Vector"), if any
  std::vector<std::string> blockArgs;
  std::vector<Type> blockArgTypes;
  std::vector<Op> body;
  // tensor.extract_slice / tensor.empty / tensor.extract / linalg.index / tensor.concat
  std::vector<IndexOperand> offsets, sizes, strides;
  int64_t dim = 0;
  // printing
  size_t srcBegin = 0, srcEnd = 0;    // span in the source text
  size_t typesBegin = 0;              // afir ops, return: where the trailing type signature starts (it ends at srcEnd)
  size_t attrInsertPos = 0;           // where "attrs = {...}" / "{...}" can be inserted (0 = none)
  std::vector<std::pair<std::string, std::string>> addedAttrs;
  int line = 0;
};

struct FuncArg {
  std::string name;
  Type type;
};

struct Func {
  std::string name;
  std::vector<FuncArg> args;
  std::vector<Type> resultTypes;
  size_t resultTypesBegin = 0, resultTypesEnd = 0;  // span of the result type(s) after "->", parentheses included (0 = none)
  std::vector<Op> ops;
  size_t attrInsertPos = 0;           // just before the body's '{'
  size_t attrDictPos = 0;             // position of the '{' of an existing "attributes {...}" (0 = none)
  std::string existingAttrs;          // text of that dictionary, braces included
  std::vector<std::pair<std::string, std::string>> addedAttrs;
  int line = 0;
};

// A transform-dialect schedule found beside the payload functions (transform.named_sequence @__transform_main ...),
// the form the reference's examples keep their tiling strategy in (examples/*/step2_transform.mlir).  It is not
// interpreted op by op: what this backend needs from it is how many index arguments it adds to the kernel
// (transform.func.add_index_args, lib/Dialect/AFIR/TransformOps/AFIRTransformOps.cpp:25-109: the tile parameters
// of the TilingData struct) and, for the record, the tile sizes and annotations it names.
struct TransformSchedule {
  std::string name;                       // @__transform_main
  int indexArgs = 0;                      // sum over transform.func.add_index_args
  std::vector<std::string> tileSizes;     // the text of every tile_sizes [...] list, in order
  std::vector<std::string> annotations;   // names given to transform.annotate ("ascendc.parallel", ...)
  size_t srcBegin = 0, srcEnd = 0;        // span of the whole op in the source text
};

struct Module {
  std::string source;
  std::map<std::string, AffineMap> mapAliases;
  std::vector<Func> funcs;
  std::vector<TransformSchedule> schedules;
  size_t moduleAttrBegin = 0, moduleAttrEnd = 0;  // span of "attributes {...}" after the module keyword (0 = none)
  // spans of the source text that printModule leaves out (a pass that removes the schedule fills this)
  std::vector<std::pair<size_t, size_t>> erasures;
  // spans [begin, end) that printModule replaces by other text (a pass that rewrites ops fills this)
  struct Replacement { size_t begin, end; std::string text; };
  std::vector<Replacement> replacements;
};

Status parseModule(const std::string &text, Module &out);
// The source text with every added attribute spliced in.
std::string printModule(const Module &m);

} // namespace front
} // namespace afir
