#include "front/shape_inference.h"

#include <algorithm>
#include <map>

namespace afir {
namespace front {

bool inferBroadcastShape(const std::vector<std::vector<int64_t>> &operands, std::vector<int64_t> &out) {
  size_t rank = 0;
  for (const auto &shape : operands) rank = std::max(rank, shape.size());
  out.assign(rank, 1);
  for (size_t pos = rank; pos-- > 0;) {
    for (const auto &shape : operands) {
      const size_t lead = rank - shape.size();  // positions this operand does not have
      if (pos < lead) continue;
      const int64_t extent = shape[pos - lead];
      if (extent == 1) continue;
      if (out[pos] < 0 || out[pos] == 1) out[pos] = extent;
      if (extent < 0) continue;
      if (out[pos] != extent) return false;
    }
  }
  return true;
}

bool inferConcatShape(const std::vector<std::vector<int64_t>> &operands, int64_t axis, std::vector<int64_t> &out) {
  if (operands.empty()) return false;
  const size_t rank = operands[0].size();
  for (const auto &shape : operands)
    if (shape.size() != rank) return false;
  if (axis < 0 || static_cast<size_t>(axis) >= rank) return false;
  out.assign(rank, 0);  // 0 = nothing seen yet at a position that is not the axis
  for (const auto &shape : operands)
    for (size_t j = 0; j < rank; ++j) {
      if (shape[j] < 0) out[j] = -1;
      else if (j == static_cast<size_t>(axis)) { if (out[j] >= 0) out[j] += shape[j]; }
      else if (out[j] == 0) out[j] = shape[j];
      else if (out[j] >= 0 && out[j] != shape[j]) return false;
    }
  return true;
}

bool inferReducedShape(const std::vector<int64_t> &operand, int64_t axis, std::vector<int64_t> &out) {
  if (axis < 0 || static_cast<size_t>(axis) >= operand.size()) return false;
  out = operand;
  out.erase(out.begin() + axis);
  return true;
}

bool joinShapes(const std::vector<int64_t> &current, const std::vector<int64_t> &inferred, std::vector<int64_t> &out) {
  if (current.size() != inferred.size()) return false;
  out.assign(current.size(), -1);
  for (size_t i = 0; i < current.size(); ++i) {
    if (current[i] < 0) out[i] = inferred[i];
    else if (inferred[i] < 0 || inferred[i] == current[i]) out[i] = current[i];
    else return false;
  }
  return true;
}

namespace {

std::string typeListText(const std::vector<Type> &types) {
  std::string s;
  for (size_t i = 0; i < types.size(); ++i) s += (i ? ", " : "") + types[i].str();
  return s;
}

bool sameType(const Type &a, const Type &b) { return a.isTensor == b.isTensor && a.dims == b.dims && a.elem == b.elem; }

// End of the text of a type signature that the parser left at `end`, possibly past trailing white space.
size_t trimmedEnd(const std::string &source, size_t begin, size_t end) {
  end = std::min(end, source.size());
  while (end > begin && (source[end - 1] == ' ' || source[end - 1] == '\t' || source[end - 1] == '\n' || source[end - 1] == '\r')) --end;
  return end;
}

} // namespace

void inferAfirShapes(Module &m, int *refined) {
  if (refined) *refined = 0;
  for (Func &f : m.funcs) {
    std::map<std::string, Type> env;  // SSA name -> its type as refined so far
    for (const FuncArg &a : f.args) env[a.name] = a.type;
    for (Op &o : f.ops) {
      if (o.name.compare(0, 5, "afir.") == 0 && o.typesBegin != 0 && o.results.size() == 1) {
        // operands print with the types their values have now
        std::vector<Type> operandTypes = o.operandTypes;
        for (size_t i = 0; i < o.operands.size() && i < operandTypes.size(); ++i) {
          const auto known = env.find(o.operands[i]);
          if (known != env.end()) operandTypes[i] = known->second;
        }
        Type result = o.resultType;
        bool ranked = result.isTensor;
        std::vector<std::vector<int64_t>> shapes;
        for (const Type &t : operandTypes) {
          ranked = ranked && t.isTensor;
          shapes.push_back(t.dims);
        }
        std::vector<int64_t> inferred, joined;
        const std::string kind = o.name.substr(5);
        const bool reduction = kind == "sum" || kind == "max" || kind == "min" || kind == "mean" || kind == "prod" || kind == "any" || kind == "all";
        bool inferredOk;
        if (kind == "concat") inferredOk = inferConcatShape(shapes, o.dim, inferred);
        else if (reduction) inferredOk = shapes.size() == 1 && inferReducedShape(shapes[0], o.dim, inferred);
        else inferredOk = inferBroadcastShape(shapes, inferred);
        if (ranked && inferredOk && joinShapes(result.dims, inferred, joined) && joined != result.dims) {
          result.dims = joined;
          if (refined) ++*refined;
        }
        bool changed = !sameType(result, o.resultType);
        for (size_t i = 0; i < operandTypes.size(); ++i) changed = changed || !sameType(operandTypes[i], o.operandTypes[i]);
        if (changed) {
          // (unary ops print their operand type without parentheses; the form found in the source is kept)
          const bool parens = o.typesBegin < m.source.size() && m.source[o.typesBegin] == '(';
          m.replacements.push_back({o.typesBegin, trimmedEnd(m.source, o.typesBegin, o.srcEnd),
                                    (parens ? "(" : "") + typeListText(operandTypes) + (parens ? ")" : "") + " -> " + result.str()});
          o.operandTypes = operandTypes;
          o.resultType = result;
        }
        env[o.results[0]] = result;
      } else if ((o.name == "return" || o.name == "func.return") && o.typesBegin != 0) {
        std::vector<Type> types = o.operandTypes;
        for (size_t i = 0; i < o.operands.size() && i < types.size(); ++i) {
          const auto known = env.find(o.operands[i]);
          if (known != env.end()) types[i] = known->second;
        }
        bool changed = false;
        for (size_t i = 0; i < types.size(); ++i) changed = changed || !sameType(types[i], o.operandTypes[i]);
        if (changed) {
          m.replacements.push_back({o.typesBegin, trimmedEnd(m.source, o.typesBegin, o.srcEnd), typeListText(types)});
          o.operandTypes = types;
        }
        // the function returns what its (first) return op returns
        if (f.resultTypesBegin != 0 && types.size() == f.resultTypes.size()) {
          bool resultChanged = false;
          for (size_t i = 0; i < types.size(); ++i) resultChanged = resultChanged || !sameType(types[i], f.resultTypes[i]);
          if (resultChanged) {
            m.replacements.push_back({f.resultTypesBegin, trimmedEnd(m.source, f.resultTypesBegin, f.resultTypesEnd),
                                      types.size() == 1 ? types[0].str() : "(" + typeListText(types) + ")"});
            f.resultTypes = types;
          }
        }
      } else if (o.results.size() == 1 && !o.resultType.elem.empty()) {
        env[o.results[0]] = o.resultType;  // (ops that print no result type leave their users' types as written)
      }
    }
  }
}

} // namespace front
} // namespace afir
