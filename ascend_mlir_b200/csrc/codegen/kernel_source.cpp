#include "codegen/kernel_source.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <sstream>

namespace afir {
namespace codegen {
namespace {

// ---- symbolic extents and strides ------------------------------------------------------------------------------
// A product  coef * f1 * f2 * ...  of TilingData fields: enough to express every extent and stride of a dense
// row-major tensor whose dims are literals or tiling fields, and to decide at generation time whether two
// neighbouring iteration dims are walked contiguously by a view (stride[d] == stride[d+1] * extent[d+1]).
constexpr const char *kRowsName = "@rows";  // the leading iteration extent after the row window (a kernel local)

struct Sym {
  int64_t coef = 0;
  std::vector<std::string> fields;  // sorted

  static Sym literal(int64_t v) { Sym s; s.coef = v; return s; }
  static Sym field(const std::string &name) { Sym s; s.coef = 1; s.fields.push_back(name); return s; }
  bool isZero() const { return coef == 0; }
  bool isLiteral() const { return fields.empty(); }
  bool isLiteral(int64_t v) const { return fields.empty() && coef == v; }
  bool operator==(const Sym &o) const { return coef == o.coef && (coef == 0 || fields == o.fields); }
};

Sym mul(const Sym &a, const Sym &b) {
  Sym r;
  r.coef = a.coef * b.coef;
  if (r.coef == 0) return r;
  r.fields = a.fields;
  r.fields.insert(r.fields.end(), b.fields.begin(), b.fields.end());
  std::sort(r.fields.begin(), r.fields.end());
  return r;
}

Sym symOf(const DimExpr &e) { return e.literal ? Sym::literal(e.value) : Sym::field(e.field); }

std::string identifier(const std::string &name) {
  std::string id;
  for (char c : name) id.push_back((std::isalnum(static_cast<unsigned char>(c)) || c == '_') ? c : '_');
  if (id.empty() || std::isdigit(static_cast<unsigned char>(id[0]))) id = "f_" + id;
  return id;
}

std::string fieldCode(const std::string &name) { return name == kRowsName ? std::string("rows0") : "t." + identifier(name); }

std::string code(const Sym &s) {
  if (s.coef == 0) return "0LL";
  std::string out;
  if (s.coef != 1 || s.fields.empty()) out = std::to_string(s.coef) + "LL";
  for (const std::string &f : s.fields) {
    if (!out.empty()) out += " * ";
    out += fieldCode(f);
  }
  return out;
}

std::string code(const DimExpr &e) { return e.literal ? std::to_string(e.value) + "LL" : "t." + identifier(e.field); }

// A view over the iteration domain, symbolically: element stride per iteration dim and the base offset as code.
struct SymView {
  int arg = -1;
  std::vector<Sym> stride;
  std::string offset;  // elements; "" = none
  Sym rowStride;       // stride of iteration dim 0 before any collapsing (what one row of the row window is worth)
};

bool buildView(const ViewSpec &v, size_t rank, SymView &out, std::string &why) {
  out = SymView();
  out.arg = v.arg;
  out.stride.assign(rank, Sym());
  Sym suffix = Sym::literal(1);
  std::vector<Sym> tensorStride(v.shape.size());
  for (int t = static_cast<int>(v.shape.size()) - 1; t >= 0; --t) {
    tensorStride[t] = suffix;
    suffix = mul(suffix, symOf(v.shape[t]));
  }
  for (size_t t = 0; t < v.shape.size(); ++t) {
    const int d = v.map.empty() ? -1 : v.map[t];
    if (d >= 0) {
      if (static_cast<size_t>(d) >= rank) { why = "a view maps to an iteration dim outside the domain"; return false; }
      if (!out.stride[d].isZero()) { why = "one iteration dim indexes two dims of the same tensor"; return false; }
      out.stride[d] = tensorStride[t];
    }
    if (!v.offset.empty()) {
      const DimExpr &o = v.offset[t];
      if (o.literal && o.value == 0) continue;
      if (!out.offset.empty()) out.offset += " + ";
      out.offset += "(" + code(o) + ") * (" + code(tensorStride[t]) + ")";
    }
  }
  out.rowStride = rank > 0 ? out.stride[0] : Sym();
  return true;
}

// Drops literal extent-1 dims and merges neighbours that every view walks contiguously (same rule as the
// launcher's collapseDomain, decided on symbols instead of numbers).
void collapse(std::vector<Sym> &extent, std::vector<SymView *> &views) {
  for (size_t d = 0; d < extent.size() && extent.size() > 1;) {
    if (extent[d].isLiteral(1)) {
      extent.erase(extent.begin() + d);
      for (SymView *v : views) v->stride.erase(v->stride.begin() + d);
    } else ++d;
  }
  for (size_t d = 0; d + 1 < extent.size();) {
    bool mergeable = true;
    for (SymView *v : views)
      if (!(v->stride[d] == mul(v->stride[d + 1], extent[d + 1]))) { mergeable = false; break; }
    if (mergeable) {
      extent[d + 1] = mul(extent[d], extent[d + 1]);
      extent.erase(extent.begin() + d);
      for (SymView *v : views) v->stride.erase(v->stride.begin() + d);
    } else ++d;
  }
}

// ---- element types ------------------------------------------------------------------------------------------------
struct TypeInfo {
  const char *pack;
  int bytes;
  bool integer;
  const char *define;  // macro the translation unit needs, or null
};

bool typeInfo(DType t, bool integersToo, TypeInfo &out) {
  switch (t) {
  case DType::F32: out = {"PackF32", 4, false, nullptr}; return true;
  case DType::F16: out = {"PackF16", 2, false, "AFIR_CG_F16"}; return true;
  case DType::BF16: out = {"PackBF16", 2, false, "AFIR_CG_BF16"}; return true;
  case DType::I32: out = {"PackI32", 4, true, nullptr}; return integersToo;
  case DType::I16: out = {"PackI16", 2, true, nullptr}; return integersToo;
  default: return false;
  }
}

// ---- the fused body as straight-line code ----------------------------------------------------------------------------
std::string operandCode(const kernels::BodySrc &s, bool integer) {
  char buf[64];
  switch (s.kind) {
  case kernels::kSrcView: return "v[" + std::to_string(s.index) + "]";
  case kernels::kSrcOp: return "r" + std::to_string(s.index);
  default:
    if (integer) {
      std::snprintf(buf, sizeof(buf), "P::constantInt(%d)", s.ivalue);
    } else {
      unsigned int bits;
      std::memcpy(&bits, &s.value, sizeof(bits));
      std::snprintf(buf, sizeof(buf), "P::constant(__uint_as_float(0x%08xu))", bits);  // the exact bits, not a decimal
    }
    return buf;
  }
}

const char *opName(int op) {
  switch (op) {
  case kernels::kOpAdd: return "add";
  case kernels::kOpSub: return "sub";
  case kernels::kOpMul: return "mul";
  case kernels::kOpDiv: return "div";
  case kernels::kOpMax: return "max";
  default: return "min";
  }
}

std::string bodyStruct(const std::string &name, const kernels::BodyProgram &b, int numViews, bool integer) {
  std::ostringstream os;
  os << "struct " << name << " {\n"
     << "  static constexpr int kViews = " << std::max(1, numViews) << ";\n"
     << "  static constexpr bool kInterpreted = false;\n"
     << "  template <class P> __device__ __forceinline__ static P eval(const P *v, const afir::kernels::BodyProgram &) {\n";
  for (int i = 0; i < b.numOps; ++i)
    os << "    const P r" << i << " = P::" << opName(b.ops[i].op) << "(" << operandCode(b.ops[i].a, integer) << ", "
       << operandCode(b.ops[i].b, integer) << ");\n";
  if (b.numOps == 0) os << "    return v[0];\n";
  else os << "    return r" << (b.numOps - 1) << ";\n";
  os << "  }\n};\n";
  return os.str();
}

// ---- common text ---------------------------------------------------------------------------------------------------
std::string tilingStruct(const LaunchDescriptor &d) {
  std::ostringstream os;
  os << "// all-int64 TilingData: the descriptor's fields in order, then the words the runtime fills in at launch\n"
     << "struct TilingData {\n";
  for (const TilingField &f : d.tiling) os << "  long long " << identifier(f.name) << ";\n";
  os << "  long long afir_row_begin, afir_row_end;  // window of the leading iteration dim; afir_row_end < 0 = all of it\n"
     << "  long long afir_p0, afir_p1, afir_p2, afir_p3, afir_p4, afir_p5;  // launch plan\n"
     << "};\n";
  return os.str();
}

std::string signature(const LaunchDescriptor &d, const std::string &entry, const char *bounds) {
  std::ostringstream os;
  os << "extern \"C\" __global__ void " << bounds << " " << entry << "(";
  for (int i = 0; i < d.numInputs; ++i) os << "const void *arg" << i << ", ";
  for (int i = 0; i < d.numOutputs; ++i) os << "void *arg" << (d.numInputs + i) << ", ";
  os << "void *workspace, const __grid_constant__ TilingData t)";
  return os.str();
}

// The same parameters as signature(), for a device function, and the matching argument list of a call.
std::string parameterList(const LaunchDescriptor &d) {
  std::ostringstream os;
  for (int i = 0; i < d.numInputs; ++i) os << "const void *arg" << i << ", ";
  for (int i = 0; i < d.numOutputs; ++i) os << "void *arg" << (d.numInputs + i) << ", ";
  os << "void *workspace, const TilingData &t";
  return os.str();
}

std::string argumentList(const LaunchDescriptor &d) {
  std::ostringstream os;
  for (int i = 0; i < d.numInputs + d.numOutputs; ++i) os << "arg" << i << ", ";
  os << "workspace, t";
  return os.str();
}

// `dependent`: the kernel starts with gridDependencyPrologue() and its module carries the marker kernel, so the
// runtime launches it with programmatic stream serialisation.  Gather kernels do not: with one short CTA per tile
// the prologue's two instructions, executed by every CTA, were measured to cost more than the overlap gains.
std::string rowWindowPrologue(bool dependent = true) {
  return std::string(dependent ? "  gridDependencyPrologue();\n" : "") +
         "  if (t.afir_row_end >= 0 && t.afir_row_end <= t.afir_row_begin) return;  // empty row window\n"
         "  const long long rowb = t.afir_row_end >= 0 ? t.afir_row_begin : 0;\n"
         "  (void)workspace; (void)rowb;\n";
}

std::string rowsDecl(const DimExpr &leading) {
  return "    const long long rows0 = t.afir_row_end >= 0 ? t.afir_row_end - t.afir_row_begin : " + code(leading) + ";\n";
}

// (const char *)argN + (offset + rowb * rowStride) * elemBytes
std::string baseCode(const SymView &v, int elemBytes, bool isConst) {
  std::string elems = v.offset;
  if (!v.rowStride.isZero()) {
    if (!elems.empty()) elems += " + ";
    elems += "rowb * (" + code(v.rowStride) + ")";
  }
  std::string p = std::string(isConst ? "static_cast<const char *>(arg" : "static_cast<char *>(arg") + std::to_string(v.arg) + ")";
  if (elems.empty()) return p;
  return p + " + (" + elems + ") * " + std::to_string(elemBytes);
}

std::string aligned16(const std::string &ptr) { return "((reinterpret_cast<unsigned long long>(" + ptr + ") & 15ull) == 0ull)"; }

const char *kPreamble =
    "// Generated for one fused group; the loops are the function templates of kernels/*_skel.cuh.\n"
    "using namespace afir::kernels;\n\n";
const char *kDependencyMarker =
    "// Tells the runtime that every kernel of this module begins with gridDependencyPrologue().\n"
    "extern \"C\" __global__ void afir_waits_for_grid_dependencies() {}\n\n";

// ---- elementwise / broadcast / split / concat ------------------------------------------------------------------------
bool emitElementwiseGroup(const LaunchDescriptor &d, const GroupSpec &g, size_t index, const TypeInfo &ti, std::ostringstream &bodies,
                          std::ostringstream &kernel, std::string &why, int &blockCtasPerSm) {
  const size_t rank = g.domain.size();
  if (rank == 0) { why = "empty iteration domain"; return false; }
  if (g.loads.empty() || g.loads.size() > static_cast<size_t>(kernels::kMaxViews)) { why = "group loads no view or too many"; return false; }
  std::vector<SymView> views(g.loads.size() + 1);
  for (size_t i = 0; i < g.loads.size(); ++i) {
    if (g.loads[i].dtype != d.dtype) { why = "a load differs from the group element type"; return false; }
    if (!buildView(g.loads[i], rank, views[i], why)) return false;
  }
  if (!buildView(g.store, rank, views.back(), why)) return false;
  const bool leadingIsOne = g.domain[0].literal && g.domain[0].value == 1;
  std::vector<Sym> extent(rank);
  for (size_t k = 0; k < rank; ++k) extent[k] = symOf(g.domain[k]);
  if (!leadingIsOne) extent[0] = Sym::field(kRowsName);
  std::vector<SymView *> all;
  for (SymView &v : views) all.push_back(&v);
  collapse(extent, all);
  if (extent.size() > 3) { why = "iteration space keeps more than three dims after collapsing"; return false; }
  while (extent.size() < 3) {
    extent.insert(extent.begin(), Sym::literal(1));
    for (SymView *v : all) v->stride.insert(v->stride.begin(), Sym());
  }
  const bool innerIsOne = extent[2].isLiteral(1);
  SymView &store = views.back();
  if (!store.stride[2].isLiteral(1) && !innerIsOne) { why = "the store is not contiguous along the inner dim"; return false; }
  // A view whose unit stride runs along the middle dim is read through a transpose (out[n, m] = f(a[m, n], ...)):
  // such a group gets the register-block loop beside the element-wise one.
  bool transposedGroup = false;
  for (size_t i = 0; i < g.loads.size(); ++i) {
    if (innerIsOne) views[i].stride[2] = Sym::literal(1);
    if (!views[i].stride[2].isLiteral(0) && !views[i].stride[2].isLiteral(1)) {
      if (!views[i].stride[1].isLiteral(1)) {
        why = "an operand is contiguous along neither of the two inner dims";
        return false;
      }
      transposedGroup = true;
    }
  }
  if (transposedGroup && g.body.numOps == 0) {
    why = "a bare permutation runs on the library's transpose kernels";
    return false;
  }
  if (transposedGroup) {
    // CTAs per SM the kernel is compiled for.  Three (a budget of 80 registers) where the blocks of all views fit
    // without spilling: a view that is not constant along the inner dim holds 16 bytes per block row, 8 rows of 16-bit
    // elements or 4 of 32-bit ones.  Two (up to 128 registers) for wider groups.  Measured on (a^T + b) * c, f16
    // 8192 x 8192: 64.0 us with the budget of 80 stated against 68.3 us without (the run-time compiler then settled
    // on 73 registers, three CTAs per SM as well, and issued fewer loads ahead of their first use).
    int fullViews = 0;
    for (size_t i = 0; i < g.loads.size(); ++i)
      if (!views[i].stride[2].isLiteral(0)) ++fullViews;
    const int ctas = fullViews <= (ti.bytes == 2 ? 2 : 5) ? 3 : 2;
    blockCtasPerSm = blockCtasPerSm == 0 ? ctas : std::min(blockCtasPerSm, ctas);
  }
  const int ve = 16 / ti.bytes;
  const std::string bodyName = "FusedBody" + std::to_string(index);
  bodies << bodyStruct(bodyName, g.body, static_cast<int>(g.loads.size()), ti.integer) << "\n";

  std::ostringstream &os = kernel;
  os << "  {  // group " << index << "\n" << rowsDecl(g.domain[0]);
  os << "    EwParams prm = {};\n";
  os << "    const long long d0 = " << code(extent[0]) << ", d1 = " << code(extent[1]) << ", d2 = " << code(extent[2]) << ";\n";
  std::string vec = "d2 % " + std::to_string(ve) + " == 0";
  for (size_t i = 0; i < g.loads.size(); ++i) {
    const SymView &v = views[i];
    os << "    prm.vbase[" << i << "] = " << baseCode(v, ti.bytes, true) << ";\n";
    os << "    prm.vs0[" << i << "] = " << code(v.stride[0]) << "; prm.vs1[" << i << "] = " << code(v.stride[1]) << "; prm.vs2[" << i
       << "] = " << code(v.stride[2]) << ";\n";
    if (v.stride[2].isLiteral(1))
      vec += " && " + aligned16("prm.vbase[" + std::to_string(i) + "]") + " && prm.vs0[" + std::to_string(i) + "] % " + std::to_string(ve) +
             " == 0 && prm.vs1[" + std::to_string(i) + "] % " + std::to_string(ve) + " == 0";
  }
  os << "    prm.obase = " << baseCode(store, ti.bytes, false) << ";\n";
  os << "    prm.os0 = " << code(store.stride[0]) << "; prm.os1 = " << code(store.stride[1]) << ";\n";
  vec += " && " + aligned16("prm.obase") + " && prm.os0 % " + std::to_string(ve) + " == 0 && prm.os1 % " + std::to_string(ve) + " == 0";
  if (transposedGroup) vec = "false";  // (the transposed view has no 16-byte pieces along the inner dim)
  os << "    const bool vec = " << vec << ";\n";
  os << "    const long long vpr = vec ? d2 / " << ve << " : d2;\n";
  os << "    prm.vecPerRow = static_cast<unsigned int>(vpr);\n"
     << "    prm.d1 = static_cast<unsigned int>(d1);\n"

     << "    prm.totalVec = static_cast<unsigned int>(d0 * d1 * vpr);\n"
     << "    prm.flat = (d0 == 1 && d1 == 1) ? 1 : 0;\n"
     << "    prm.numViews = " << g.loads.size() << ";\n"
     << "    const unsigned int tileVecs = blockDim.x * 2u;\n"
     << "    prm.numTiles = (prm.totalVec + tileVecs - 1u) / tileVecs;\n";
  if (transposedGroup) {
    // The register-block loop when the launch has its CTA shape (256 threads) and everything is aligned for 16-byte
    // row pieces: row-major views along their rows, transposed views along theirs; else element by element.
    const int tileRows = 2 * 4 * ve, tileCols = 4 * 8 * ve;
    std::string ok = "blockDim.x == 256u && " + aligned16("prm.obase") + " && prm.os0 % " + std::to_string(ve) + " == 0 && prm.os1 % " +
                     std::to_string(ve) + " == 0";
    os << "    EbParams bp = {};\n";
    for (size_t i = 0; i < g.loads.size(); ++i) {
      const SymView &v = views[i];
      const char *kind = v.stride[2].isLiteral(1) ? "kViewRowMajor" : v.stride[2].isLiteral(0) ? "kViewInnerBroadcast" : "kViewTransposed";
      os << "    bp.vbase[" << i << "] = prm.vbase[" << i << "]; bp.s0[" << i << "] = prm.vs0[" << i << "]; bp.s1[" << i << "] = prm.vs1[" << i
         << "]; bp.s2[" << i << "] = prm.vs2[" << i << "]; bp.kind[" << i << "] = " << kind << ";\n";
      const std::string n = std::to_string(i), e = std::to_string(ve);
      if (v.stride[2].isLiteral(1)) ok += " && " + aligned16("prm.vbase[" + n + "]") + " && prm.vs0[" + n + "] % " + e + " == 0 && prm.vs1[" + n + "] % " + e + " == 0";
      else if (!v.stride[2].isLiteral(0)) ok += " && " + aligned16("prm.vbase[" + n + "]") + " && prm.vs0[" + n + "] % " + e + " == 0 && prm.vs2[" + n + "] % " + e + " == 0";
    }
    os << "    bp.numViews = " << g.loads.size() << "; bp.obase = prm.obase; bp.os0 = prm.os0; bp.os1 = prm.os1; bp.d1 = d1; bp.d2 = d2;\n"
       << "    bp.tilesX = static_cast<unsigned int>((d2 + " << (tileCols - 1) << ") / " << tileCols << ");\n"
       << "    bp.tilesY = static_cast<unsigned int>((d1 + " << (tileRows - 1) << ") / " << tileRows << ");\n"
       << "    bp.numTiles = static_cast<unsigned long long>(d0) * bp.tilesX * bp.tilesY;\n"
       << "    if (" << ok << ") elementwiseBlocksTiles<" << ti.pack << ", " << bodyName << ", " << g.loads.size() << ">(bp);\n"
       << "    else elementwiseTiles<" << ti.pack << ", " << bodyName << ", 2, false, false, true>(prm);\n"
       << "  }\n";
    return true;
  }
  os << "    if (vec) elementwiseTiles<" << ti.pack << ", " << bodyName << ", 2, true, false, true>(prm);\n"
     << "    else elementwiseTiles<" << ti.pack << ", " << bodyName << ", 2, false, false, true>(prm);\n"
     << "  }\n";
  return true;
}

GeneratedKernel generateElementwise(const LaunchDescriptor &d) {
  GeneratedKernel out;
  TypeInfo ti;
  if (!typeInfo(d.dtype, true, ti)) { out.whyNot = "element type"; return out; }
  if (d.groups.empty()) { out.whyNot = "no groups"; return out; }
  std::ostringstream bodies, kernel;
  int blockCtasPerSm = 0;  // 0 = no group with a transposed operand
  for (size_t i = 0; i < d.groups.size(); ++i)
    if (!emitElementwiseGroup(d, d.groups[i], i, ti, bodies, kernel, out.whyNot, blockCtasPerSm)) return out;
  const bool usesBlocks = blockCtasPerSm > 0;
  out.hasTransposedOperand = usesBlocks;
  std::ostringstream src;
  src << (usesBlocks ? "#include \"kernels/elementwise_blocks_skel.cuh\"\n" : "#include \"kernels/elementwise_skel.cuh\"\n") << kPreamble << kDependencyMarker
      << (usesBlocks ? "// Tells the runtime that this module's kernel is launched with CTAs of 256 threads.\nextern \"C\" __global__ void afir_ctas_of_256_threads() {}\n\n" : "")
      << tilingStruct(d) << "\n" << bodies.str()
      // (a kernel with the register-block loop is launched with 256 threads, like the library's instantiations)
      << signature(d, d.kernel, !usesBlocks ? "__launch_bounds__(512)" : blockCtasPerSm == 3 ? "__launch_bounds__(256, 3)" : "__launch_bounds__(256)")
      << " {\n" << rowWindowPrologue()
      << kernel.str() << "}\n";
  out.source = src.str();
  out.entry = d.kernel;
  if (ti.define) out.defines.push_back(ti.define);
  out.supported = true;
  return out;
}

// ---- broadcast + elementwise + row reduction -----------------------------------------------------------------------------
GeneratedKernel generateRowReduce(const LaunchDescriptor &d) {
  GeneratedKernel out;
  TypeInfo ti;
  if (!typeInfo(d.dtype, false, ti)) { out.whyNot = "row reductions compute in f32, f16 or bf16"; return out; }
  if (d.groups.size() != 1) { out.whyNot = "one group per row-reduction kernel"; return out; }
  const GroupSpec &g = d.groups[0];
  const size_t rank = g.domain.size();
  if (rank < 2) { out.whyNot = "row reduction needs a [rows..., cols] domain"; return out; }
  if (g.loads.empty() || g.loads.size() > static_cast<size_t>(kernels::kMaxViews)) { out.whyNot = "group loads no view or too many"; return out; }
  std::vector<SymView> views(g.loads.size() + 1);
  for (size_t i = 0; i < g.loads.size(); ++i) {
    if (g.loads[i].dtype != d.dtype) { out.whyNot = "a load differs from the group element type"; return out; }
    if (!buildView(g.loads[i], rank, views[i], out.whyNot)) return out;
  }
  if (!buildView(g.store, rank, views.back(), out.whyNot)) return out;
  SymView &store = views.back();
  if (!store.stride.back().isZero()) { out.whyNot = "the reduced dim indexes the output"; return out; }
  const bool leadingIsOne = g.domain[0].literal && g.domain[0].value == 1;
  std::vector<Sym> outer(rank - 1);
  for (size_t k = 0; k + 1 < rank; ++k) outer[k] = symOf(g.domain[k]);
  if (!leadingIsOne) outer[0] = Sym::field(kRowsName);
  std::vector<Sym> colStride;
  std::vector<SymView *> all;
  for (SymView &v : views) {
    colStride.push_back(v.stride.back());
    v.stride.pop_back();
    all.push_back(&v);
  }
  collapse(outer, all);
  if (outer.size() != 1) { out.whyNot = "leading dims do not collapse to one row dim"; return out; }
  if (!store.stride[0].isLiteral(1) && !outer[0].isLiteral(1)) { out.whyNot = "output rows are not contiguous"; return out; }
  int streamed = -1, numStreamed = 0;
  for (size_t i = 0; i < g.loads.size(); ++i) {
    if (colStride[i].isLiteral(1)) { streamed = static_cast<int>(i); ++numStreamed; }
    else if (!colStride[i].isLiteral(0)) { out.whyNot = "an operand is not contiguous along the reduced dim"; return out; }
  }
  const std::string cols = code(symOf(g.domain.back()));
  const std::string rows = code(outer[0]);
  const int ve = 16 / ti.bytes;

  std::ostringstream src;
  src << "#include \"kernels/row_reduce_skel.cuh\"\n" << kPreamble << kDependencyMarker << tilingStruct(d) << "\n"
      << bodyStruct("FusedBody0", g.body, static_cast<int>(g.loads.size()), false) << "\n";

  // entry 1: one team of lanes per row (and per column slice), plain loads
  src << signature(d, d.kernel, "__launch_bounds__(512)") << " {\n" << rowWindowPrologue() << "  {\n" << rowsDecl(g.domain[0]);
  src << "    RrParams prm = {};\n";
  for (size_t i = 0; i < g.loads.size(); ++i)
    src << "    prm.vbase[" << i << "] = " << baseCode(views[i], ti.bytes, true) << "; prm.rowStride[" << i << "] = " << code(views[i].stride[0])
        << "; prm.colStride[" << i << "] = " << (colStride[i].isLiteral(1) ? 1 : 0) << ";\n";
  src << "    prm.numViews = " << g.loads.size() << ";\n"
      << "    prm.rows = " << rows << ";\n"
      << "    const bool vec = t.afir_p0 != 0;\n"
      << "    prm.vecPerRow = static_cast<unsigned int>((" << cols << ") / (vec ? " << ve << " : 1));\n"
      << "    prm.slices = static_cast<int>(t.afir_p1);\n"
      << "    prm.vecPerSlice = static_cast<unsigned int>(t.afir_p2);\n"
      << "    prm.lanesPerRow = static_cast<int>(t.afir_p3);\n"
      << "    prm.partial = reinterpret_cast<float *>(static_cast<char *>(workspace) + 256);\n"
      << "    prm.out = " << baseCode(store, ti.bytes, false) << ";\n"
      << "    if (vec) rowReduceTeams<" << ti.pack << ", FusedBody0, true>(prm);\n"
      << "    else rowReduceTeams<" << ti.pack << ", FusedBody0, false>(prm);\n"
      << "  }\n}\n\n";

  // entry 2: the bulk-copy staged loop, when exactly one view is streamed along the reduced dim
  if (numStreamed == 1) {
    src << signature(d, d.kernel + "__staged", "__launch_bounds__(512, 1)") << " {\n"
        << "  extern __shared__ __align__(128) unsigned char streamSmem[];\n"
        << rowWindowPrologue() << "  {\n" << rowsDecl(g.domain[0]);
    src << "    RrStreamParams sp = {};\n";
    for (size_t i = 0; i < g.loads.size(); ++i) {
      if (static_cast<int>(i) == streamed)
        src << "    sp.stream = " << baseCode(views[i], ti.bytes, true) << "; sp.streamRowStride = " << code(views[i].stride[0]) << ";\n";
      else
        src << "    sp.bcast[" << i << "] = " << baseCode(views[i], ti.bytes, true) << "; sp.bcastRowStride[" << i << "] = " << code(views[i].stride[0])
            << ";\n";
    }
    src << "    sp.streamViewIndex = " << streamed << ";\n"
        << "    sp.numViews = " << g.loads.size() << ";\n"
        << "    sp.rows = " << rows << ";\n"
        << "    sp.rowBytes = static_cast<unsigned int>((" << cols << ") * " << ti.bytes << ");\n"
        << "    sp.stages = static_cast<int>(t.afir_p0);\n"
        << "    sp.chunkBytes = static_cast<unsigned int>(t.afir_p1);\n"
        << "    sp.out = " << baseCode(store, ti.bytes, false) << ";\n"
        << "    sp.status = reinterpret_cast<unsigned int *>(static_cast<char *>(workspace) + 8);\n"
        << "    rowReduceStream<" << ti.pack << ", FusedBody0>(sp, streamSmem);\n"
        << "  }\n}\n\n";
    out.hasStaged = true;
  }

  // entry 3: adds the column slices' partial sums in slice order
  src << signature(d, d.kernel + "__finalize", "") << " {\n" << rowWindowPrologue() << "  {\n" << rowsDecl(g.domain[0])
      << "    rowReduceFinalize<" << ti.pack << ">(reinterpret_cast<const float *>(static_cast<char *>(workspace) + 256), " << baseCode(store, ti.bytes, false)
      << ", " << rows << ", static_cast<int>(t.afir_p1));\n"
      << "  }\n}\n";
  out.hasFinalize = true;

  out.source = src.str();
  out.entry = d.kernel;
  if (ti.define) out.defines.push_back(ti.define);
  out.supported = true;
  return out;
}

// ---- row gather + elementwise ---------------------------------------------------------------------------------------------
GeneratedKernel generateGatherRows(const LaunchDescriptor &d) {
  GeneratedKernel out;
  TypeInfo ti;
  if (!typeInfo(d.dtype, false, ti)) { out.whyNot = "gather groups compute in f32, f16 or bf16"; return out; }
  if (d.groups.size() != 1) { out.whyNot = "one group per gather kernel"; return out; }
  const GroupSpec &g = d.groups[0];
  if (g.gatherAxis != 0) { out.whyNot = "column gathers run on the prebuilt kernel"; return out; }
  if (g.domain.size() != 2) { out.whyNot = "gather needs a [rows, cols] domain"; return out; }
  if (g.loads.empty() || g.loads.size() > static_cast<size_t>(kernels::kMaxViews)) { out.whyNot = "group loads no view or too many"; return out; }
  const ViewSpec &table = g.loads[0];
  if (table.shape.size() != 2 || table.dtype != d.dtype) { out.whyNot = "the table is a 2-D tensor of the group element type"; return out; }
  if (g.indices.dtype != DType::I32 && g.indices.dtype != DType::I64) { out.whyNot = "indices are i32 or i64"; return out; }
  std::vector<SymView> views(g.loads.size() + 1);
  for (size_t i = 1; i < g.loads.size(); ++i) {
    if (g.loads[i].dtype != d.dtype) { out.whyNot = "a load differs from the group element type"; return out; }
    if (!buildView(g.loads[i], 2, views[i], out.whyNot)) return out;
    if (!views[i].stride[1].isLiteral(0) && !views[i].stride[1].isLiteral(1)) { out.whyNot = "an operand is not contiguous along the inner dim"; return out; }
  }
  SymView &store = views.back();
  if (!buildView(g.store, 2, store, out.whyNot)) return out;
  if (!store.stride[1].isLiteral(1)) { out.whyNot = "the output is not contiguous along the inner dim"; return out; }
  const int ve = 16 / ti.bytes;
  const int indexBytes = g.indices.dtype == DType::I64 ? 8 : 4;
  const std::string cols = code(symOf(g.domain[1]));
  const std::string tcols = code(symOf(table.shape[1]));

  std::ostringstream src;
  src << "#include \"kernels/gather_skel.cuh\"\n" << kPreamble << tilingStruct(d) << "\n"
      << bodyStruct("FusedBody0", g.body, static_cast<int>(g.loads.size()), false) << "\n"
      // The loop body once, as a function template: PAIR = the variant with two vectors per thread in flight is
      // compiled in.  That variant needs about twice the registers of the others, and a kernel's register count is
      // that of its hungriest path, so the entry used by default (<kernel>__one) leaves it out and keeps every warp
      // slot of the SM usable (measured on the 262 144 x 256 bf16 gather: 40 registers and 66 % of the warp slots
      // active with all three paths in one kernel, 22 registers and 85 % without).
      << "template <bool PAIR>\n__device__ __forceinline__ void " << d.kernel << "__body(" << parameterList(d) << ") {\n"
      << rowWindowPrologue(false) << "  {\n" << rowsDecl(g.domain[0]);
  src << "    GaParams prm = {};\n"
      << "    prm.table = static_cast<const char *>(arg" << table.arg << ");\n"
      << "    prm.tableRows = " << code(symOf(table.shape[0])) << "; prm.tableCols = " << tcols << "; prm.tableRowStride = " << tcols << ";\n"
      << "    prm.indices = static_cast<const char *>(arg" << g.indices.arg << ") + rowb * " << indexBytes << ";\n"
      << "    prm.index64 = " << (indexBytes == 8 ? 1 : 0) << ";\n";
  std::string vec = "cols % " + std::to_string(ve) + " == 0 && " + aligned16("prm.table") + " && prm.tableRowStride % " + std::to_string(ve) + " == 0";
  for (size_t i = 1; i < g.loads.size(); ++i) {
    src << "    prm.vbase[" << i << "] = " << baseCode(views[i], ti.bytes, true) << "; prm.rowStride[" << i << "] = " << code(views[i].stride[0])
        << "; prm.colStride[" << i << "] = " << (views[i].stride[1].isLiteral(1) ? 1 : 0) << ";\n";
    if (views[i].stride[1].isLiteral(1))
      vec += " && " + aligned16("prm.vbase[" + std::to_string(i) + "]") + " && prm.rowStride[" + std::to_string(i) + "] % " + std::to_string(ve) + " == 0";
  }
  vec += " && " + aligned16("prm.out") + " && prm.outRowStride % " + std::to_string(ve) + " == 0";
  src << "    prm.numViews = " << g.loads.size() << ";\n"
      << "    prm.out = " << baseCode(store, ti.bytes, false) << ";\n"
      << "    prm.outRowStride = " << code(store.stride[0]) << ";\n"
      << "    prm.status = static_cast<unsigned long long *>(workspace);\n"
      << "    const long long cols = " << cols << ";\n"
      << "    const bool vec = " << vec << ";\n"
      << "    prm.vecPerRow = static_cast<unsigned int>(vec ? cols / " << ve << " : cols);\n"
      << "    // multiply-shift constants of the division by vecPerRow, prepared by the host for both access widths\n"
      << "    const unsigned long long mg = static_cast<unsigned long long>(vec ? t.afir_p1 : t.afir_p2);\n"
      << "    prm.divVpr.magic = static_cast<unsigned int>(mg); prm.divVpr.shift = static_cast<unsigned int>(mg >> 32); prm.divVpr.divisor = prm.vecPerRow;\n"
      << "    prm.totalVec = static_cast<unsigned int>(rows0 * prm.vecPerRow);\n"
      << "    const unsigned int inFlight = t.afir_p0 == 1 ? 1u : 2u;\n"
      << "    if (!vec) gatherRowsTiles<" << ti.pack << ", FusedBody0, 2, false>(prm);\n"
      << "    else if (!PAIR || inFlight == 1u) gatherRowsTiles<" << ti.pack << ", FusedBody0, 1, true>(prm);\n"
      << "    else gatherRowsTiles<" << ti.pack << ", FusedBody0, 2, true>(prm);\n"
      << "  }\n}\n\n"
      << signature(d, d.kernel, "__launch_bounds__(512)") << " {\n  " << d.kernel << "__body<true>(" << argumentList(d) << ");\n}\n\n"
      << "// one vector per thread in flight (the default plan): the entry the runtime launches unless the plan asks for two\n"
      << signature(d, d.kernel + "__one", "__launch_bounds__(512)") << " {\n  " << d.kernel << "__body<false>(" << argumentList(d) << ");\n}\n";
  out.source = src.str();
  out.entry = d.kernel;
  out.hasSingleVectorEntry = true;
  if (ti.define) out.defines.push_back(ti.define);
  out.supported = true;
  return out;
}

} // namespace

GeneratedKernel generateKernelSource(const LaunchDescriptor &d) {
  GeneratedKernel out;
  if (d.kernel.empty() || identifier(d.kernel) != d.kernel) {
    out.whyNot = "the kernel name is not a C identifier";
    return out;
  }
  for (size_t i = 0; i < d.tiling.size(); ++i)
    for (size_t j = i + 1; j < d.tiling.size(); ++j)
      if (identifier(d.tiling[i].name) == identifier(d.tiling[j].name)) {
        out.whyNot = "two tiling fields map to one identifier";
        return out;
      }
  switch (d.kernelClass) {
  case KernelClass::Elementwise: return generateElementwise(d);
  case KernelClass::RowReduce: return generateRowReduce(d);
  case KernelClass::Gather: return generateGatherRows(d);
  case KernelClass::Transpose: out.whyNot = "a bare permutation has no body to generate: it runs on the prebuilt transpose kernel"; return out;
  case KernelClass::Matmul: out.whyNot = "the matmul group is the hand-written tcgen05 kernel of the library"; return out;
  }
  out.whyNot = "unknown kernel class";
  return out;
}

} // namespace codegen
} // namespace afir
