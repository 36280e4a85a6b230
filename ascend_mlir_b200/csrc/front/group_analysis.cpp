#include "front/group_analysis.h"

#include <algorithm>
#include <cmath>

namespace afir {
namespace front {
namespace {

// ---- symbolic model ----------------------------------------------------------------------------------
struct Dim {
  bool lit = true;
  int64_t v = 0;
  std::string field;
  bool operator==(const Dim &o) const { return lit == o.lit && (lit ? v == o.v : field == o.field); }
  json::Value toJson() const { return lit ? json::Value(v) : json::Value(field); }
};
Dim litDim(int64_t v) { Dim d; d.v = v; return d; }
Dim fieldDim(const std::string &f) { Dim d; d.lit = false; d.field = f; return d; }

enum class ViewKind { Argument, Gathered, Accumulator };

struct View {
  ViewKind kind = ViewKind::Argument;
  int arg = -1;
  std::string dtype;
  std::vector<Dim> shape;   // of the whole argument
  std::vector<int> map;     // tensor dim -> index dim of the owning expression, -1 = fixed
  std::vector<Dim> offset;  // per tensor dim
  bool sameAs(const View &o) const { return kind == o.kind && arg == o.arg && map == o.map && offset == o.offset; }
};

struct Src {
  enum Kind { ViewValue, OpValue, Constant } kind = Constant;
  int index = 0;
  double value = 0.0;
};

struct BodyOp {
  std::string op;  // addf subf mulf divf maximumf minimumf
  Src a, b;
};

// A tensor value as an elementwise function of its own index space.
struct Elementwise {
  std::vector<Dim> extents;
  std::string dtype;
  std::vector<View> views;
  std::vector<BodyOp> ops;
  Src result;
  // gather (views[0] is the gathered table value)
  bool hasGather = false;
  int gatherAxis = -1, indicesArg = -1;
  std::string indicesType;
  Dim indicesLen;
  // matmul (views[0] is the accumulator)
  bool hasMatmul = false;
  bool transB = false;  // linalg.matmul_transpose_b: B is [N, K]
  int aArg = -1, bArg = -1, initArg = -1;
  std::string inType;
  Dim M, N, K;
};

struct Value {
  enum Kind { None, Index, Scalar, Tensor, Empty, Fill, Reduce, Concat } kind = None;
  Dim index;
  double scalar = 0.0;
  Elementwise ew;                 // Tensor; Reduce: the summand over [rows..., cols]
  std::vector<Dim> extents;       // Empty / Fill / Reduce result
  std::vector<Elementwise> parts; // Concat along dim 0
  std::string dtype;
};

struct Env {
  std::map<std::string, Value> values;
};

Status err(const Op &op, const std::string &msg) { return Status::error("line " + std::to_string(op.line) + ": " + op.name + ": " + msg); }

std::vector<Dim> typeExtents(const Type &t, int arg) {
  std::vector<Dim> out;
  for (size_t d = 0; d < t.dims.size(); ++d)
    out.push_back(t.dims[d] >= 0 ? litDim(t.dims[d]) : fieldDim("dim_arg" + std::to_string(arg) + "_" + std::to_string(d)));
  return out;
}

int addView(Elementwise &e, const View &v) {
  for (size_t i = 0; i < e.views.size(); ++i)
    if (e.views[i].sameAs(v)) return static_cast<int>(i);
  e.views.push_back(v);
  return static_cast<int>(e.views.size()) - 1;
}

// Inlines `src` (an expression over its own index space) into `dst` (over an iteration space), where
// index dim r of src is iteration dim map.results[r] (or the constant 0).  Returns where src's value lives.
Status inlineInto(Elementwise &dst, const Elementwise &src, const AffineMap &map, const Op &op, Src &out) {
  const bool identity = [&] {
    if (map.results.size() != src.extents.size()) return false;
    for (size_t r = 0; r < map.results.size(); ++r)
      if (map.results[r] != static_cast<int>(r)) return false;
    return true;
  }();
  if (map.results.size() != src.extents.size()) return err(op, "indexing map rank differs from the operand rank");
  std::vector<int> viewRemap(src.views.size());
  for (size_t i = 0; i < src.views.size(); ++i) {
    View v = src.views[i];
    if (v.kind != ViewKind::Argument) {
      if (!identity) return err(op, "a gathered or accumulated operand must be read with the identity map");
      if (!dst.views.empty() && !(dst.views[0].kind == v.kind)) return err(op, "cannot combine this operand with the group built so far");
    }
    for (int &m : v.map)
      if (m >= 0) m = map.results[m];
    if (v.kind != ViewKind::Argument) {
      if (!dst.views.empty() && dst.views[0].kind == v.kind) { viewRemap[i] = 0; continue; }
      if (!dst.views.empty()) return err(op, "the gathered / accumulated value must be the first operand of the fused group");
    }
    viewRemap[i] = addView(dst, v);
  }
  if (src.hasGather) {
    dst.hasGather = true;
    dst.gatherAxis = src.gatherAxis;
    dst.indicesArg = src.indicesArg;
    dst.indicesType = src.indicesType;
    dst.indicesLen = src.indicesLen;
  }
  if (src.hasMatmul) {
    dst.hasMatmul = true;
    dst.aArg = src.aArg; dst.bArg = src.bArg; dst.initArg = src.initArg;
    dst.inType = src.inType; dst.M = src.M; dst.N = src.N; dst.K = src.K;
    dst.transB = src.transB;
  }
  // Ops are appended with their operands renumbered; an op the group already holds (the same producer read by two
  // consumers, e.g. abs(x) = max(x, 0 - x)) is reused instead of being computed twice.
  std::vector<int> opRemap(src.ops.size(), -1);
  auto remap = [&](Src s) {
    if (s.kind == Src::ViewValue) s.index = viewRemap[s.index];
    else if (s.kind == Src::OpValue) s.index = opRemap[s.index];
    return s;
  };
  auto sameSrc = [](const Src &x, const Src &y) {
    return x.kind == y.kind && (x.kind == Src::Constant ? x.value == y.value : x.index == y.index);
  };
  for (size_t i = 0; i < src.ops.size(); ++i) {
    const BodyOp b{src.ops[i].op, remap(src.ops[i].a), remap(src.ops[i].b)};
    int found = -1;
    for (size_t j = 0; j < dst.ops.size() && found < 0; ++j)
      if (dst.ops[j].op == b.op && sameSrc(dst.ops[j].a, b.a) && sameSrc(dst.ops[j].b, b.b)) found = static_cast<int>(j);
    if (found < 0) {
      dst.ops.push_back(b);
      found = static_cast<int>(dst.ops.size()) - 1;
    }
    opRemap[i] = found;
  }
  out = remap(src.result);
  return Status::success();
}

Elementwise argumentTensor(int arg, const Type &t) {
  Elementwise e;
  e.extents = typeExtents(t, arg);
  e.dtype = t.elem;
  View v;
  v.arg = arg;
  v.dtype = t.elem;
  v.shape = e.extents;
  for (size_t d = 0; d < t.dims.size(); ++d) v.map.push_back(static_cast<int>(d));
  v.offset.assign(t.dims.size(), litDim(0));
  e.views.push_back(v);
  e.result.kind = Src::ViewValue;
  e.result.index = 0;
  return e;
}

// Body op names are the float spellings internally; integer groups are renamed when the body is emitted.
std::string arithName(const std::string &op) {
  if (op == "arith.addf" || op == "arith.addi" || op == "afir.add") return "addf";
  if (op == "arith.subf" || op == "arith.subi" || op == "afir.sub") return "subf";
  if (op == "arith.mulf" || op == "arith.muli" || op == "afir.mul") return "mulf";
  if (op == "arith.divf" || op == "arith.divsi" || op == "afir.div" || op == "afir.truediv") return "divf";
  if (op == "afir.maximum") return "maximumf";
  if (op == "afir.minimum") return "minimumf";
  if (op == "arith.maximumf" || op == "arith.maxsi") return "maximumf";
  if (op == "arith.minimumf" || op == "arith.minsi") return "minimumf";
  return "";
}

Status resolveIndex(const IndexOperand &io, const Env &env, const Op &op, Dim &out) {
  if (io.literal) { out = litDim(io.value); return Status::success(); }
  auto it = env.values.find(io.ssa);
  if (it == env.values.end() || it->second.kind != Value::Index) return err(op, "'%" + io.ssa + "' is not a known index value");
  out = it->second.index;
  return Status::success();
}

// ---- linalg.generic ----------------------------------------------------------------------------------------
struct LocalValue {
  enum Kind { Data, IterIndex, IndexCast } kind = Data;
  Src src;
  int dim = 0;       // IterIndex
  int blockArg = 0;  // IndexCast of this block argument
};

Status evalGeneric(const Op &g, size_t opIndex, const Env &env, GroupAnalysis &ga, Value &result) {
  const size_t numOuts = g.operands.size() - static_cast<size_t>(g.numIns);
  if (numOuts != 1) return err(g, "exactly one output is supported");
  const AffineMap &outMap = g.maps.back();
  const int rank = static_cast<int>(g.iterators.size());
  int numReduce = 0;
  for (const auto &it : g.iterators) numReduce += it == "reduction" ? 1 : 0;
  if (numReduce > 1 || (numReduce == 1 && g.iterators.back() != "reduction")) return err(g, "only a single, innermost reduction dim is supported");
  for (size_t r = 0; r < outMap.results.size(); ++r)
    if (outMap.results[r] != static_cast<int>(r)) return err(g, "the output must be written with an identity (or leading-dims) map");
  if (static_cast<int>(outMap.results.size()) != rank - numReduce) return err(g, "output rank does not match the parallel dims");

  // iteration extents: from the output, the reduced dim from whichever input spans it
  auto outIt = env.values.find(g.operands.back());
  if (outIt == env.values.end()) return err(g, "unknown output operand");
  std::vector<Dim> extents;
  if (outIt->second.kind == Value::Tensor) extents = outIt->second.ew.extents;
  else if (outIt->second.kind == Value::Empty || outIt->second.kind == Value::Fill) extents = outIt->second.extents;
  else return err(g, "unsupported output operand");
  if (static_cast<int>(extents.size()) != rank - numReduce) return err(g, "output operand rank mismatch");

  Elementwise e;
  e.dtype = g.operandTypes.back().elem;
  std::vector<Src> blockSrc(g.operands.size());
  std::vector<bool> isIndexInput(g.operands.size(), false);
  Dim reducedExtent;
  bool haveReduced = false;
  for (int i = 0; i < g.numIns; ++i) {
    auto it = env.values.find(g.operands[i]);
    if (it == env.values.end()) return err(g, "unknown operand '%" + g.operands[i] + "'");
    // an integer input whose element is turned into an index by the body is the index vector of a gather;
    // any other integer input is ordinary data of an integer group
    bool castToIndex = false;
    for (const Op &b : g.body)
      castToIndex = castToIndex || (b.name == "arith.index_cast" && !b.operands.empty() && static_cast<size_t>(i) < g.blockArgs.size() &&
                                    b.operands[0] == g.blockArgs[i]);
    if (castToIndex) {
      isIndexInput[i] = true;
      continue;
    }
    if (it->second.kind != Value::Tensor) return err(g, "operand '%" + g.operands[i] + "' is not an elementwise-computable tensor");
    const Elementwise &src = it->second.ew;
    if (numReduce && !haveReduced)
      for (size_t r = 0; r < g.maps[i].results.size(); ++r)
        if (g.maps[i].results[r] == rank - 1) { reducedExtent = src.extents[r]; haveReduced = true; }
    if (Status s = inlineInto(e, src, g.maps[i], g, blockSrc[i]); !s) return s;
  }
  if (numReduce) {
    if (!haveReduced) return err(g, "no input spans the reduced dim");
    extents.push_back(reducedExtent);
  }
  e.extents = extents;

  // body
  std::map<std::string, LocalValue> local;
  for (size_t i = 0; i < g.blockArgs.size(); ++i) {
    LocalValue lv;
    lv.src = blockSrc[i];
    local[g.blockArgs[i]] = lv;
  }
  const std::string accName = g.blockArgs.back();
  bool sawAccumulate = false, sawConversion = false;
  Src yielded;
  bool haveYield = false;
  auto lookup = [&](const std::string &name, LocalValue &out) -> Status {
    auto l = local.find(name);
    if (l != local.end()) { out = l->second; return Status::success(); }
    auto o = env.values.find(name);
    if (o != env.values.end() && o->second.kind == Value::Scalar) {
      out = LocalValue();
      out.src.kind = Src::Constant;
      out.src.value = o->second.scalar;
      return Status::success();
    }
    return err(g, "body uses unknown value '%" + name + "'");
  };
  for (const Op &b : g.body) {
    if (b.name == "linalg.yield") {
      LocalValue v;
      if (Status s = lookup(b.operands[0], v); !s) return s;
      yielded = v.src;
      haveYield = true;
    } else if (b.name == "arith.constant") {
      // a scalar constant defined inside the body (the reference's relu example writes its zero there)
      LocalValue lv;
      lv.src.kind = Src::Constant;
      lv.src.value = b.constIsFloat ? b.constFloat : static_cast<double>(b.constInt);
      local[b.results[0]] = lv;
    } else if (b.name == "linalg.index") {
      LocalValue lv;
      lv.kind = LocalValue::IterIndex;
      lv.dim = static_cast<int>(b.dim);
      local[b.results[0]] = lv;
    } else if (b.name == "arith.index_cast") {
      LocalValue lv;
      lv.kind = LocalValue::IndexCast;
      auto pos = std::find(g.blockArgs.begin(), g.blockArgs.end(), b.operands[0]);
      if (pos == g.blockArgs.end()) return err(g, "index_cast of a value that is not an input element");
      lv.blockArg = static_cast<int>(pos - g.blockArgs.begin());
      local[b.results[0]] = lv;
    } else if (b.name == "arith.extf" || b.name == "arith.truncf") {
      // width changes around an f32-accumulated matmul: the epilogue computes in f32 and the final type is the
      // output's; they carry the value through unchanged here
      LocalValue v;
      if (Status s = lookup(b.operands[0], v); !s) return s;
      local[b.results[0]] = v;
      sawConversion = true;
    } else if (b.name == "tensor.extract") {
      // gather: out[i, j] = T[i, idx[j]] (column form) or T[idx[i], j] (row form)
      auto t = env.values.find(b.operands[0]);
      if (t == env.values.end() || t->second.kind != Value::Tensor) return err(g, "tensor.extract from an unknown tensor");
      const Elementwise &table = t->second.ew;
      if (rank != 2 || b.offsets.size() != 2 || table.extents.size() != 2) return err(g, "only 2-D gathers are supported");
      if (table.views.size() != 1 || table.views[0].kind != ViewKind::Argument || table.hasGather || table.hasMatmul)
        return err(g, "the gathered tensor must be a function argument with optional elementwise pre-ops");
      const View &tv = table.views[0];
      for (size_t d = 0; d < 2; ++d)
        if (tv.map[d] != static_cast<int>(d) || !(tv.offset[d] == litDim(0))) return err(g, "the gathered tensor must be read whole");
      LocalValue p[2];
      for (int k = 0; k < 2; ++k) {
        if (b.offsets[k].literal) return err(g, "constant gather coordinates are not supported");
        if (Status s = lookup(b.offsets[k].ssa, p[k]); !s) return s;
      }
      int axis;
      if (p[0].kind == LocalValue::IterIndex && p[0].dim == 0 && p[1].kind == LocalValue::IndexCast) axis = 1;
      else if (p[1].kind == LocalValue::IterIndex && p[1].dim == 1 && p[0].kind == LocalValue::IndexCast) axis = 0;
      else return err(g, "gather coordinates must be one linalg.index and one index_cast of an index input");
      const int idxOperand = p[axis == 1 ? 1 : 0].blockArg;
      if (idxOperand >= g.numIns || !isIndexInput[idxOperand]) return err(g, "gather index must come from an integer input");
      const AffineMap &im = g.maps[idxOperand];
      if (im.results.size() != 1 || im.results[0] != (axis == 1 ? 1 : 0)) return err(g, "the index vector must follow the gathered axis of the output");
      auto iv = env.values.find(g.operands[idxOperand]);
      if (iv == env.values.end() || iv->second.kind != Value::Tensor || iv->second.ew.views.size() != 1 || !iv->second.ew.ops.empty())
        return err(g, "the index vector must be a function argument");
      View gv = tv;
      gv.kind = ViewKind::Gathered;
      if (!e.views.empty()) {
        // the already-fused form (what --fuse-gather-elementwise produces: the gather generic also reads the
        // broadcast extras of its post-ops): the gathered value must be view 0, so the views registered for the
        // other inputs move up by one
        if (e.views[0].kind != ViewKind::Argument || e.hasGather || e.hasMatmul) return err(g, "only one gather per fused group");
        auto shift = [](Src &src) { if (src.kind == Src::ViewValue) ++src.index; };
        for (auto &kv : local) shift(kv.second.src);
        for (BodyOp &op : e.ops) { shift(op.a); shift(op.b); }
        e.views.insert(e.views.begin(), gv);
      } else {
        e.views.push_back(gv);
      }
      e.hasGather = true;
      e.gatherAxis = axis;
      e.indicesArg = iv->second.ew.views[0].arg;
      e.indicesType = g.operandTypes[idxOperand].elem;
      e.indicesLen = iv->second.ew.extents[0];
      // pre-ops of the table commute with the gather: they run on the gathered value
      for (const BodyOp &pre : table.ops) e.ops.push_back(pre);
      LocalValue lv;
      lv.src = table.result;
      local[b.results[0]] = lv;
      ga.opAttrs[opIndex].push_back({axis == 1 ? "gather_dim" : "embedding_dim", std::to_string(axis == 1 ? 1 : 0) + " : i64"});
    } else {
      const std::string name = arithName(b.name);
      if (name.empty()) return err(g, "unsupported body op '" + b.name + "'");
      LocalValue a, c;
      if (Status s = lookup(b.operands[0], a); !s) return s;
      if (Status s = lookup(b.operands[1], c); !s) return s;
      if (a.kind != LocalValue::Data || c.kind != LocalValue::Data) return err(g, "arithmetic on index values is not supported");
      if (numReduce && (b.operands[0] == accName || b.operands[1] == accName)) {
        if (name != "addf" || sawAccumulate) return err(g, "only a single sum reduction is supported");
        sawAccumulate = true;
        LocalValue lv;
        lv.src = b.operands[0] == accName ? c.src : a.src;  // the summand
        local[b.results[0]] = lv;
        continue;
      }
      e.ops.push_back({name, a.src, c.src});
      LocalValue lv;
      lv.src.kind = Src::OpValue;
      lv.src.index = static_cast<int>(e.ops.size()) - 1;
      local[b.results[0]] = lv;
    }
  }
  if (!haveYield) return err(g, "body has no linalg.yield");
  e.result = yielded;
  if (e.views.empty()) return err(g, "a group with no tensor inputs is not supported");
  if (sawConversion && !e.hasMatmul) return err(g, "arith.extf / arith.truncf are only supported in a matmul epilogue");

  if (numReduce) {
    if (!sawAccumulate) return err(g, "reduction body must add the input to the accumulator");
    if (outIt->second.kind != Value::Fill || outIt->second.scalar != 0.0) return err(g, "the reduction must start from a zero fill");
    result.kind = Value::Reduce;
    result.ew = e;
    result.extents.assign(extents.begin(), extents.end() - 1);
    result.dtype = e.dtype;
    return Status::success();
  }
  result.kind = Value::Tensor;
  result.ew = e;
  result.dtype = e.dtype;
  return Status::success();
}

#include "front/group_emit.inc"

} // namespace

Status analyzeFunction(const Module &module, const Func &func, GroupAnalysis &out) {
  (void)module;
  out = GroupAnalysis();
  Env env;
  for (size_t a = 0; a < func.args.size(); ++a) {
    Value v;
    if (func.args[a].type.isTensor) {
      v.kind = Value::Tensor;
      v.ew = argumentTensor(static_cast<int>(a), func.args[a].type);
      v.dtype = func.args[a].type.elem;
    } else {
      return Status::error("function '" + func.name + "': only tensor arguments are supported");
    }
    env.values[func.args[a].name] = v;
  }
  std::string returned;
  for (size_t i = 0; i < func.ops.size(); ++i) {
    const Op &op = func.ops[i];
    Value v;
    if (Status s = evalOp(op, i, env, out, v, returned); !s) return s;
    if (!op.results.empty()) env.values[op.results[0]] = v;
  }
  if (returned.empty()) return Status::error("function '" + func.name + "' returns nothing");
  auto it = env.values.find(returned);
  if (it == env.values.end()) return Status::error("function '" + func.name + "' returns an unknown value");
  return emitGroup(func, it->second, out);
}

} // namespace front
} // namespace afir
