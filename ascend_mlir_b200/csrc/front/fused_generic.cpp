#include "front/fused_generic.h"

#include <cstdio>
#include <sstream>

namespace afir {
namespace front {
namespace {

std::string floatLiteral(double v) {
  char buf[64];
  std::snprintf(buf, sizeof(buf), "%.6e", v);
  return buf;
}

bool isIntegerElem(const std::string &e) { return !e.empty() && e[0] == 'i'; }

// The view covers its whole argument: no slice offsets and the argument's own shape.
bool wholeArgument(const json::Value &view, const Type &type) {
  if (const json::Value *off = view.find("offset"))
    if (off->isArray())
      for (const auto &o : off->asArray())
        if (!(o.isInt() && o.asInt() == 0)) return false;
  const json::Value *shape = view.find("shape");
  if (!shape || !shape->isArray() || shape->asArray().size() != type.dims.size()) return false;
  for (size_t d = 0; d < type.dims.size(); ++d) {
    const json::Value &s = shape->asArray()[d];
    if (type.dims[d] >= 0 ? !(s.isInt() && s.asInt() == type.dims[d]) : !s.isString()) return false;
  }
  return true;
}

std::string mapText(const json::Value &view, size_t rank) {
  AffineMap m;
  m.numDims = static_cast<int>(rank);
  if (const json::Value *map = view.find("map"))
    for (const auto &r : map->asArray()) m.results.push_back(static_cast<int>(r.asInt()));
  return m.str();
}

} // namespace

bool fuseGenericsInPlace(Module &module, const Func &func, const GroupAnalysis &ga, std::string &why) {
  const json::Value &d = ga.descriptor;
  const std::string kclass = d.getString("kernel_class", "");
  if (kclass != "elementwise" && kclass != "row_reduce" && kclass != "gather") { why = "the group is not an elementwise, reduction or gather chain"; return false; }
  if (d.find("groups")) { why = "the function holds several groups (split / concat)"; return false; }
  std::vector<const Op *> generics;
  for (const Op &o : func.ops)
    if (o.name == "linalg.generic") generics.push_back(&o);
  if (generics.size() < 2) { why = "nothing to fuse"; return false; }
  const Op &last = *generics.back();
  if (last.results.size() != 1 || last.numIns >= static_cast<int>(last.operands.size())) { why = "the last generic has no result"; return false; }
  const json::Value *loads = d.find("loads"), *store = d.find("store"), *body = d.find("body"), *domain = d.find("domain");
  if (!loads || !store || !domain) { why = "descriptor without views"; return false; }
  const size_t rank = domain->asArray().size();
  const int numInputs = static_cast<int>(d.getInt("num_inputs", 0));
  const std::string elem = d.getString("dtype", "f32");
  const bool gather = kclass == "gather";
  const json::Value *gatherInfo = d.find("gather");
  if (gather && (!gatherInfo || rank != 2)) { why = "gather without its description"; return false; }

  // operands of the fused generic: (gather: the index vector first,) then every loaded view that is a whole argument
  std::vector<std::string> operandNames, operandTypes, maps, blockArgs;
  std::vector<std::string> viewValue(loads->asArray().size());  // body name of view k
  int gatherAxis = -1;
  std::string tableName, tableType, indexElem;
  if (gather) {
    gatherAxis = static_cast<int>(gatherInfo->getInt("axis", 1));
    const json::Value *idx = gatherInfo->find("indices");
    const int idxArg = idx ? static_cast<int>(idx->getInt("arg", -1)) : -1;
    if (idxArg < 0 || idxArg >= static_cast<int>(func.args.size())) { why = "gather without an index argument"; return false; }
    indexElem = func.args[idxArg].type.elem;
    operandNames.push_back("%" + func.args[idxArg].name);
    operandTypes.push_back(func.args[idxArg].type.str());
    AffineMap im;
    im.numDims = 2;
    im.results.push_back(gatherAxis == 1 ? 1 : 0);
    maps.push_back(im.str());
    blockArgs.push_back("%idx: " + indexElem);
  }
  for (size_t k = 0; k < loads->asArray().size(); ++k) {
    const json::Value &v = loads->asArray()[k];
    const int arg = static_cast<int>(v.getInt("arg", -1));
    if (arg < 0 || arg >= numInputs || arg >= static_cast<int>(func.args.size())) { why = "a view does not read a function argument"; return false; }
    if (gather && k == 0) {  // the table: read through tensor.extract inside the body
      if (!wholeArgument(v, func.args[arg].type)) { why = "the gathered tensor is a slice"; return false; }
      tableName = "%" + func.args[arg].name;
      tableType = func.args[arg].type.str();
      viewValue[k] = "%gathered";
      continue;
    }
    if (!wholeArgument(v, func.args[arg].type)) { why = "a view is a slice of its argument"; return false; }
    operandNames.push_back("%" + func.args[arg].name);
    operandTypes.push_back(func.args[arg].type.str());
    maps.push_back(mapText(v, rank));
    viewValue[k] = "%in" + std::to_string(k);
    blockArgs.push_back(viewValue[k] + ": " + elem);
  }
  maps.push_back(mapText(*store, rank));
  blockArgs.push_back("%acc: " + elem);

  std::ostringstream os;
  os << "%" << last.results[0] << " = linalg.generic {indexing_maps = [";
  for (size_t i = 0; i < maps.size(); ++i) os << (i ? ", " : "") << maps[i];
  os << "], iterator_types = [";
  for (size_t k = 0; k < rank; ++k) os << (k ? ", " : "") << (kclass == "row_reduce" && k + 1 == rank ? "\"reduction\"" : "\"parallel\"");
  os << "]";
  if (gather) os << ", " << (gatherAxis == 1 ? "gather_dim = 1 : i64" : "embedding_dim = 0 : i64");
  os << "}\n        ins(";
  for (size_t i = 0; i < operandNames.size(); ++i) os << (i ? ", " : "") << operandNames[i];
  os << " : ";
  for (size_t i = 0; i < operandTypes.size(); ++i) os << (i ? ", " : "") << operandTypes[i];
  os << ") outs(%" << last.operands[last.numIns] << " : " << last.resultType.str() << ") {\n    ^bb0(";
  for (size_t i = 0; i < blockArgs.size(); ++i) os << (i ? ", " : "") << blockArgs[i];
  os << "):\n";
  if (gather) {
    os << "      %pos = linalg.index " << (gatherAxis == 1 ? 0 : 1) << " : index\n"
       << "      %picked = arith.index_cast %idx : " << indexElem << " to index\n"
       << "      %gathered = tensor.extract " << tableName << (gatherAxis == 1 ? "[%pos, %picked]" : "[%picked, %pos]") << " : " << tableType << "\n";
  }
  int constants = 0;
  auto operand = [&](const json::Value &src) -> std::string {
    if (src.isString()) {
      const std::string &s = src.asString();
      if (s[0] == 'v') return viewValue[static_cast<size_t>(std::stoi(s.substr(1)))];
      return "%f" + s.substr(1);
    }
    const std::string name = "%cst" + std::to_string(constants++);
    os << "      " << name << " = arith.constant "
       << (isIntegerElem(elem) ? std::to_string(src.asInt()) : floatLiteral(src.asDouble())) << " : " << elem << "\n";
    return name;
  };
  std::string value = viewValue.empty() ? "%acc" : viewValue[0];
  size_t numOps = 0;
  if (body && body->isArray()) {
    for (const auto &op : body->asArray()) {
      const json::Value *a = op.find("a"), *b = op.find("b");
      if (!a || !b) { why = "body op without operands"; return false; }
      const std::string av = operand(*a), bv = operand(*b);
      value = "%f" + std::to_string(numOps++);
      os << "      " << value << " = arith." << op.getString("op", "addf") << " " << av << ", " << bv << " : " << elem << "\n";
    }
  }
  if (kclass == "row_reduce") {
    os << "      %sum = arith.addf %acc, " << value << " : " << elem << "\n";
    value = "%sum";
  }
  os << "      linalg.yield " << value << " : " << elem << "\n    } -> " << last.resultType.str();

  for (size_t i = 0; i + 1 < generics.size(); ++i) module.erasures.push_back({generics[i]->srcBegin, generics[i]->srcEnd});
  module.replacements.push_back({last.srcBegin, last.srcEnd, os.str()});
  return true;
}

} // namespace front
} // namespace afir
