#include "runtime/descriptor.h"

#include <algorithm>

#include <cstring>

namespace afir {

const char *dtypeName(DType t) {
  switch (t) {
  case DType::F32: return "f32";
  case DType::F16: return "f16";
  case DType::BF16: return "bf16";
  case DType::I32: return "i32";
  case DType::I64: return "i64";
  case DType::U8: return "u8";
  case DType::I16: return "i16";
  }
  return "?";
}

bool parseDType(const std::string &s, DType &out) {
  if (s == "f32" || s == "float32") out = DType::F32;
  else if (s == "f16" || s == "float16") out = DType::F16;
  else if (s == "bf16" || s == "bfloat16") out = DType::BF16;
  else if (s == "i32" || s == "int32") out = DType::I32;
  else if (s == "i64" || s == "int64") out = DType::I64;
  else if (s == "u8" || s == "ui8" || s == "uint8") out = DType::U8;
  else if (s == "i16" || s == "int16") out = DType::I16;
  else return false;
  return true;
}

size_t dtypeBytes(DType t) {
  switch (t) {
  case DType::F32: case DType::I32: return 4;
  case DType::F16: case DType::BF16: case DType::I16: return 2;
  case DType::I64: return 8;
  case DType::U8: return 1;
  }
  return 0;
}

const char *kernelClassName(KernelClass c) {
  switch (c) {
  case KernelClass::Elementwise: return "elementwise";
  case KernelClass::RowReduce: return "row_reduce";
  case KernelClass::Gather: return "gather";
  case KernelClass::Transpose: return "transpose";
  case KernelClass::Matmul: return "matmul";
  }
  return "?";
}

size_t LaunchDescriptor::tilingBytes() const {
  size_t n = 0;
  for (const auto &f : tiling) n += static_cast<size_t>(f.bytes);
  return n;
}

namespace {

Status parseDim(const json::Value &v, DimExpr &out, const char *what) {
  if (v.isInt()) {
    out.literal = true;
    out.value = v.asInt();
    if (out.value < 0) return Status::error(std::string(what) + ": negative dimension");
    return Status::success();
  }
  if (v.isString() && !v.asString().empty()) {
    out.literal = false;
    out.field = v.asString();
    return Status::success();
  }
  return Status::error(std::string(what) + ": a dimension must be an integer or a tiling field name");
}

Status parseDimList(const json::Value *v, std::vector<DimExpr> &out, const char *what) {
  out.clear();
  if (!v) return Status::success();
  if (!v->isArray()) return Status::error(std::string(what) + " must be an array");
  for (const auto &e : v->asArray()) {
    DimExpr d;
    if (Status s = parseDim(e, d, what); !s) return s;
    out.push_back(d);
  }
  return Status::success();
}

Status parseView(const json::Value &v, DType dfltType, int numArgs, size_t domainRank, bool needMap, ViewSpec &out,
                 const char *what) {
  if (!v.isObject()) return Status::error(std::string(what) + " must be an object");
  out.arg = static_cast<int>(v.getInt("arg", -1));
  if (out.arg < 0 || out.arg >= numArgs) return Status::error(std::string(what) + ": 'arg' out of range");
  out.dtype = dfltType;
  if (const json::Value *t = v.find("dtype")) {
    if (!t->isString() || !parseDType(t->asString(), out.dtype)) return Status::error(std::string(what) + ": unknown dtype");
  }
  if (Status s = parseDimList(v.find("shape"), out.shape, what); !s) return s;
  if (out.shape.empty()) return Status::error(std::string(what) + ": 'shape' is required");
  if (Status s = parseDimList(v.find("offset"), out.offset, what); !s) return s;
  if (!out.offset.empty() && out.offset.size() != out.shape.size())
    return Status::error(std::string(what) + ": 'offset' rank differs from 'shape'");
  out.map.clear();
  if (const json::Value *m = v.find("map")) {
    if (!m->isArray()) return Status::error(std::string(what) + ": 'map' must be an array");
    for (const auto &e : m->asArray()) {
      if (!e.isInt()) return Status::error(std::string(what) + ": 'map' entries are integers");
      int64_t d = e.asInt();
      if (d < -1 || d >= static_cast<int64_t>(domainRank)) return Status::error(std::string(what) + ": 'map' entry out of range");
      out.map.push_back(static_cast<int>(d));
    }
    if (out.map.size() != out.shape.size()) return Status::error(std::string(what) + ": 'map' rank differs from 'shape'");
  } else if (needMap) {
    return Status::error(std::string(what) + ": 'map' is required");
  }
  return Status::success();
}

Status parseSrc(const json::Value &v, int numViews, int opIndex, kernels::BodySrc &out) {
  out = {};
  if (v.isNumber()) {
    out.kind = kernels::kSrcConst;
    out.value = static_cast<float>(v.asDouble());
    // integer element types read the constant from here: exact, where the float above rounds beyond 2^24
    const double d = v.asDouble();
    const long long wide = v.isInt() ? static_cast<long long>(v.asInt())
                                     : (d >= -9.2e18 && d <= 9.2e18 ? static_cast<long long>(d) : 0ll);
    out.ivalue = static_cast<int>(static_cast<unsigned int>(static_cast<unsigned long long>(wide)));  // wraps like the type
    return Status::success();
  }
  if (!v.isString() || v.asString().size() < 2) return Status::error("body operand must be \"v<k>\", \"%<k>\" or a number");
  const std::string &s = v.asString();
  char *end = nullptr;
  long idx = std::strtol(s.c_str() + 1, &end, 10);
  if (!end || *end != '\0' || idx < 0) return Status::error("bad body operand '" + s + "'");
  if (s[0] == 'v') {
    if (idx >= numViews) return Status::error("body operand '" + s + "' names a view that is not loaded");
    out.kind = kernels::kSrcView;
  } else if (s[0] == '%') {
    if (idx >= opIndex) return Status::error("body operand '" + s + "' is used before it is defined");
    out.kind = kernels::kSrcOp;
  } else {
    return Status::error("bad body operand '" + s + "'");
  }
  out.index = static_cast<int>(idx);
  return Status::success();
}

Status parseBody(const json::Value *v, int numViews, kernels::BodyProgram &out) {
  out = {};
  if (!v) return Status::success();
  if (!v->isArray()) return Status::error("'body' must be an array");
  const auto &ops = v->asArray();
  if (ops.size() > static_cast<size_t>(kernels::kMaxBodyOps))
    return Status::error("fused body has more than " + std::to_string(kernels::kMaxBodyOps) + " ops");
  for (size_t i = 0; i < ops.size(); ++i) {
    const json::Value &o = ops[i];
    if (!o.isObject()) return Status::error("body op must be an object");
    const std::string name = o.getString("op");
    int code;
    // float and (signed) integer spellings name the same op; the group's dtype decides the arithmetic
    if (name == "addf" || name == "addi" || name == "add") code = kernels::kOpAdd;
    else if (name == "subf" || name == "subi" || name == "sub") code = kernels::kOpSub;
    else if (name == "mulf" || name == "muli" || name == "mul") code = kernels::kOpMul;
    else if (name == "divf" || name == "divsi" || name == "div") code = kernels::kOpDiv;
    else if (name == "maximumf" || name == "maxsi" || name == "max") code = kernels::kOpMax;
    else if (name == "minimumf" || name == "minsi" || name == "min") code = kernels::kOpMin;
    else return Status::error("unsupported body op '" + name + "'");
    const json::Value *a = o.find("a"), *b = o.find("b");
    if (!a || !b) return Status::error("body op '" + name + "' needs operands 'a' and 'b'");
    out.ops[i].op = code;
    if (Status s = parseSrc(*a, numViews, static_cast<int>(i), out.ops[i].a); !s) return s;
    if (Status s = parseSrc(*b, numViews, static_cast<int>(i), out.ops[i].b); !s) return s;
  }
  out.numOps = static_cast<int>(ops.size());
  kernels::finishBodyProgram(out);
  return Status::success();
}

Status parseGroup(const json::Value &g, const LaunchDescriptor &d, GroupSpec &out) {
  const int numArgs = d.numInputs + d.numOutputs;
  if (Status s = parseDimList(g.find("domain"), out.domain, "domain"); !s) return s;
  if (out.domain.empty() || out.domain.size() > 8) return Status::error("'domain' must have 1 to 8 dims");
  const json::Value *loads = g.find("loads");
  if (!loads || !loads->isArray() || loads->asArray().empty()) return Status::error("'loads' must be a non-empty array");
  if (loads->asArray().size() > static_cast<size_t>(kernels::kMaxViews))
    return Status::error("more than " + std::to_string(kernels::kMaxViews) + " loaded views");
  const bool gather = d.kernelClass == KernelClass::Gather;
  size_t i = 0;
  for (const auto &lv : loads->asArray()) {
    ViewSpec v;
    const bool isTable = gather && i == 0;
    if (Status s = parseView(lv, d.dtype, numArgs, out.domain.size(), !isTable, v, "load"); !s) return s;
    out.loads.push_back(std::move(v));
    ++i;
  }
  const json::Value *store = g.find("store");
  if (!store) return Status::error("'store' is required");
  if (Status s = parseView(*store, d.dtype, numArgs, out.domain.size(), true, out.store, "store"); !s) return s;
  if (out.store.arg < d.numInputs) return Status::error("'store' must name an output argument");
  if (Status s = parseBody(g.find("body"), static_cast<int>(out.loads.size()), out.body); !s) return s;
  if (gather) {
    const json::Value *ga = g.find("gather");
    if (!ga || !ga->isObject()) return Status::error("gather groups need a 'gather' object");
    out.gatherAxis = static_cast<int>(ga->getInt("axis", -1));
    if (out.gatherAxis != 0 && out.gatherAxis != 1) return Status::error("gather axis must be 0 or 1");
    const json::Value *idx = ga->find("indices");
    if (!idx) return Status::error("gather needs 'indices'");
    if (Status s = parseView(*idx, DType::I32, numArgs, out.domain.size(), false, out.indices, "indices"); !s) return s;
    if (out.indices.dtype != DType::I32 && out.indices.dtype != DType::I64) return Status::error("gather indices must be i32 or i64");
    if (out.domain.size() != 2) return Status::error("gather groups iterate over a 2-D domain");
  }
  return Status::success();
}

} // namespace

Status parseDescriptorJson(const json::Value &root, LaunchDescriptor &out) {
  out = LaunchDescriptor();
  if (!root.isObject()) return Status::error("launch descriptor must be a JSON object");
  if (root.getString("format") != "afir-cuda-launch") return Status::error("not an afir-cuda-launch descriptor");
  if (root.getInt("version", 0) != 1) return Status::error("unsupported launch descriptor version");
  const std::string arch = root.getString("arch", "sm_100a");
  if (arch != "sm_100a") return Status::error("descriptor targets '" + arch + "', this library is sm_100a only");
  out.kernel = root.getString("kernel");
  if (out.kernel.empty()) return Status::error("descriptor has no kernel name");
  const std::string cls = root.getString("kernel_class");
  if (cls == "elementwise") out.kernelClass = KernelClass::Elementwise;
  else if (cls == "row_reduce") out.kernelClass = KernelClass::RowReduce;
  else if (cls == "gather") out.kernelClass = KernelClass::Gather;
  else if (cls == "transpose") out.kernelClass = KernelClass::Transpose;
  else if (cls == "matmul") out.kernelClass = KernelClass::Matmul;
  else return Status::error("unknown kernel_class '" + cls + "'");
  if (!parseDType(root.getString("dtype", "f32"), out.dtype)) return Status::error("unknown dtype");
  out.numInputs = static_cast<int>(root.getInt("num_inputs", -1));
  out.numOutputs = static_cast<int>(root.getInt("num_outputs", -1));
  if (out.numInputs < 0 || out.numOutputs <= 0 || out.numInputs + out.numOutputs > 16)
    return Status::error("invalid num_inputs/num_outputs");

  if (const json::Value *t = root.find("tiling")) {
    if (!t->isArray()) return Status::error("'tiling' must be an array");
    for (const auto &e : t->asArray()) {
      TilingField f;
      if (e.isString()) f.name = e.asString();
      else if (e.isObject()) {
        f.name = e.getString("name");
        const std::string ty = e.getString("type", "int64");
        if (ty == "int64" || ty == "int64_t") f.bytes = 8;
        else if (ty == "int32" || ty == "int32_t") f.bytes = 4;
        else return Status::error("tiling field '" + f.name + "' has unsupported type '" + ty + "'");
      }
      if (f.name.empty()) return Status::error("tiling field without a name");
      for (const auto &prev : out.tiling)
        if (prev.name == f.name) return Status::error("duplicate tiling field '" + f.name + "'");
      out.tiling.push_back(f);
    }
  }
  if (const json::Value *l = root.find("launch"); l && l->isObject()) {
    out.ctaThreadsField = l->getString("cta_threads");
    out.unrollField = l->getString("unroll");
    out.splitColsField = l->getString("split_cols");
    out.stagesField = l->getString("stages");
    out.teamLanesField = l->getString("team_lanes");
    out.bulkCopyField = l->getString("bulk_copy");
    out.streamStagesField = l->getString("stream_stages");
    out.streamChunkField = l->getString("stream_chunk_bytes");
    out.warpRowsField = l->getString("warp_rows");
    out.ctasPerSmField = l->getString("ctas_per_sm");
    out.tileKernelField = l->getString("tile_kernel");
    out.tileOrderField = l->getString("tile_order");
    out.variantField = l->getString("variant");
    out.streamRowsField = l->getString("stream_rows");
    out.streamWarpsField = l->getString("stream_warps");
  }

  if (out.kernelClass == KernelClass::Matmul) {
    const json::Value *m = root.find("matmul");
    if (!m || !m->isObject()) return Status::error("matmul descriptors need a 'matmul' object");
    MatmulSpec &ms = out.matmul;
    const int numArgs = out.numInputs + out.numOutputs;
    ms.aArg = static_cast<int>(m->getInt("a", 0));
    ms.bArg = static_cast<int>(m->getInt("b", 1));
    ms.biasArg = static_cast<int>(m->getInt("bias", -1));
    ms.outArg = static_cast<int>(m->getInt("out", numArgs - 1));
    if (ms.aArg < 0 || ms.aArg >= numArgs || ms.bArg < 0 || ms.bArg >= numArgs || ms.biasArg >= numArgs ||
        ms.outArg < out.numInputs || ms.outArg >= numArgs)
      return Status::error("matmul argument index out of range");
    if (!parseDType(m->getString("in_dtype", "bf16"), ms.inType) || !parseDType(m->getString("out_dtype", "bf16"), ms.outType) ||
        !parseDType(m->getString("bias_dtype", "bf16"), ms.biasType))
      return Status::error("matmul: unknown dtype");
    const std::string epi = m->getString("epilogue", "None");
    if (epi == "None") ms.epilogue = kernels::kEpiNone;
    else if (epi == "BiasAdd") ms.epilogue = kernels::kEpiBiasAdd;
    else if (epi == "BiasAddLeakyRelu") ms.epilogue = kernels::kEpiBiasAddLeakyRelu;
    else if (epi == "BiasAddRelu") ms.epilogue = kernels::kEpiBiasAddRelu;
    else return Status::error("matmul: unknown epilogue kind '" + epi + "'");
    if (ms.epilogue != kernels::kEpiNone && ms.biasArg < 0) return Status::error("matmul epilogue needs a bias argument");
    ms.alpha = m->getDouble("alpha", 0.0);
    ms.transposeB = m->getBool("transpose_b", false);
    const json::Value *dm = m->find("m"), *dn = m->find("n"), *dk = m->find("k");
    if (!dm || !dn || !dk) return Status::error("matmul needs 'm', 'n' and 'k'");
    if (Status s = parseDim(*dm, ms.m, "matmul.m"); !s) return s;
    if (Status s = parseDim(*dn, ms.n, "matmul.n"); !s) return s;
    if (Status s = parseDim(*dk, ms.k, "matmul.k"); !s) return s;
    return Status::success();
  }

  if (const json::Value *gs = root.find("groups")) {
    if (!gs->isArray() || gs->asArray().empty()) return Status::error("'groups' must be a non-empty array");
    for (const auto &g : gs->asArray()) {
      GroupSpec spec;
      if (Status s = parseGroup(g, out, spec); !s) return s;
      out.groups.push_back(std::move(spec));
    }
  } else {
    GroupSpec spec;
    if (Status s = parseGroup(root, out, spec); !s) return s;
    out.groups.push_back(std::move(spec));
  }
  return Status::success();
}

std::string embeddedDescriptorJson(const std::string &text) {
  const size_t begin = text.find(kEmbeddedDescriptorBegin);
  if (begin == std::string::npos) return std::string();
  const size_t end = text.find(kEmbeddedDescriptorEnd, begin);
  if (end == std::string::npos) return std::string();
  std::string json;
  size_t pos = text.find('\n', begin);
  while (pos != std::string::npos && pos + 1 < end) {
    const size_t lineEnd = text.find('\n', pos + 1);
    std::string line = text.substr(pos + 1, (lineEnd == std::string::npos ? end : std::min(lineEnd, end)) - pos - 1);
    if (line.compare(0, 3, "// ") == 0) json += line.substr(3);
    else if (line.compare(0, 2, "//") == 0) json += line.substr(2);
    pos = lineEnd;
    if (lineEnd == std::string::npos || lineEnd >= end) break;
  }
  return json;
}

std::string embedDescriptorComment(const std::string &compactJson) {
  return std::string(kEmbeddedDescriptorBegin) + "\n// " + compactJson + "\n" + kEmbeddedDescriptorEnd + "\n";
}

Status parseDescriptorBinary(const uint8_t *data, size_t len, LaunchDescriptor &out) {
  if (!data || len == 0) return Status::error("binary data is required");
  std::string text;
  if (len >= 12 && std::memcmp(data, "AFCU", 4) == 0) {
    uint32_t version, jsonLen;
    std::memcpy(&version, data + 4, 4);
    std::memcpy(&jsonLen, data + 8, 4);
    if (version != kContainerVersion && version != kContainerVersionWithCode) return Status::error("unsupported kernel container version");
    if (static_cast<size_t>(jsonLen) + 12 > len) return Status::error("truncated kernel container");
    text.assign(reinterpret_cast<const char *>(data + 12), jsonLen);
  } else {
    size_t i = 0;
    while (i < len && (data[i] == ' ' || data[i] == '\n' || data[i] == '\t' || data[i] == '\r')) ++i;
    if (i < len && data[i] == '{') {
      text.assign(reinterpret_cast<const char *>(data), len);
    } else {
      // a kernel source file with its descriptor in the leading comment block
      text = embeddedDescriptorJson(std::string(reinterpret_cast<const char *>(data), len));
      if (text.empty()) return Status::error("kernel binary is neither an AFCU container, a launch descriptor nor a kernel source with one embedded");
    }
  }
  json::Value root;
  std::string err;
  if (!json::parse(text, root, err)) return Status::error("launch descriptor: " + err);
  return parseDescriptorJson(root, out);
}

std::vector<uint8_t> wrapDescriptorContainer(const std::string &jsonText, const std::vector<uint8_t> &cubin, const std::string &source) {
  const bool withCode = !cubin.empty() || !source.empty();
  std::vector<uint8_t> out(12 + jsonText.size() + (withCode ? 8 + cubin.size() + source.size() : 0));
  std::memcpy(out.data(), "AFCU", 4);
  const uint32_t version = withCode ? kContainerVersionWithCode : kContainerVersion, n = static_cast<uint32_t>(jsonText.size());
  std::memcpy(out.data() + 4, &version, 4);
  std::memcpy(out.data() + 8, &n, 4);
  std::memcpy(out.data() + 12, jsonText.data(), jsonText.size());
  if (withCode) {
    size_t off = 12 + jsonText.size();
    const uint32_t cubinLen = static_cast<uint32_t>(cubin.size()), sourceLen = static_cast<uint32_t>(source.size());
    std::memcpy(out.data() + off, &cubinLen, 4);
    if (cubinLen) std::memcpy(out.data() + off + 4, cubin.data(), cubin.size());
    off += 4 + cubin.size();
    std::memcpy(out.data() + off, &sourceLen, 4);
    if (sourceLen) std::memcpy(out.data() + off + 4, source.data(), source.size());
  }
  return out;
}

ContainerCode containerCode(const uint8_t *data, size_t len) {
  ContainerCode code;
  if (!data || len < 12 || std::memcmp(data, "AFCU", 4) != 0) return code;
  uint32_t version, jsonLen;
  std::memcpy(&version, data + 4, 4);
  std::memcpy(&jsonLen, data + 8, 4);
  if (version != kContainerVersionWithCode) return code;
  size_t off = 12 + static_cast<size_t>(jsonLen);
  uint32_t cubinLen = 0, sourceLen = 0;
  if (off + 4 > len) return code;
  std::memcpy(&cubinLen, data + off, 4);
  if (off + 4 + cubinLen + 4 > len) return code;
  const uint8_t *cubin = data + off + 4;
  off += 4 + cubinLen;
  std::memcpy(&sourceLen, data + off, 4);
  if (off + 4 + sourceLen > len) return code;
  code.cubin = cubin;
  code.cubinLen = cubinLen;
  code.source = reinterpret_cast<const char *>(data + off + 4);
  code.sourceLen = sourceLen;
  return code;
}

Status unpackTiling(const LaunchDescriptor &d, const uint8_t *bytes, size_t len, std::map<std::string, int64_t> &out) {
  out.clear();
  const size_t want = d.tilingBytes();
  if (len != want)
    return Status::error("tiling data is " + std::to_string(len) + " bytes, kernel '" + d.kernel + "' expects " +
                         std::to_string(want));
  if (want && !bytes) return Status::error("tiling data is required");
  size_t off = 0;
  for (const auto &f : d.tiling) {
    int64_t v;
    if (f.bytes == 8) std::memcpy(&v, bytes + off, 8);
    else {
      int32_t w;
      std::memcpy(&w, bytes + off, 4);
      v = w;
    }
    out[f.name] = v;
    off += static_cast<size_t>(f.bytes);
  }
  return Status::success();
}

} // namespace afir
