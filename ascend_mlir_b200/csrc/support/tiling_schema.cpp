#include "support/tiling_schema.h"

#include <cstring>
#include <fstream>
#include <iterator>
#include <sstream>

namespace afir {

Status readFileBytes(const std::string &path, std::vector<uint8_t> &out) {
  std::ifstream is(path, std::ios::binary);
  if (!is) return Status::error("cannot open " + path);
  out.assign(std::istreambuf_iterator<char>(is), std::istreambuf_iterator<char>());
  return Status::success();
}

Status readFileText(const std::string &path, std::string &out) {
  std::ifstream is(path);
  if (!is) return Status::error("cannot open " + path);
  out.assign(std::istreambuf_iterator<char>(is), std::istreambuf_iterator<char>());
  return Status::success();
}

Status TilingSchema::fromJsonFile(const std::string &path, TilingSchema &out) {
  std::string text;
  if (Status s = readFileText(path, text); !s) return Status::error("cannot open '" + path + "'");
  json::Value root;
  std::string err;
  if (!json::parse(text, root, err)) return Status::error("JSON parse error in '" + path + "': " + err);
  return fromJsonValue(root, path, out);
}

Status TilingSchema::fromJsonValue(const json::Value &root, const std::string &origin, TilingSchema &out) {
  out = TilingSchema();
  if (!root.isObject()) return Status::error("'" + origin + "': root must be a JSON object");
  const json::Value *params = root.find("tiling_params");
  if (!params || !params->isArray()) return Status::error("'" + origin + "': missing 'tiling_params' array");
  for (const auto &e : params->asArray()) {
    if (!e.isObject()) return Status::error("'" + origin + "': tiling_params entry is not an object");
    TilingSchemaField f;
    f.name = e.getString("name");
    if (f.name.empty()) return Status::error("'" + origin + "': tiling_params entry missing 'name'");
    f.type = e.getString("type", "int64");
    out.fields_.push_back(std::move(f));
  }
  return Status::success();
}

Status TilingSchema::pack(const std::vector<std::pair<std::string, int64_t>> &params, std::vector<uint8_t> &bytes) const {
  bytes.clear();
  if (params.size() != fields_.size()) {
    std::string msg = "tiling param count mismatch: got " + std::to_string(params.size()) + ", expected " +
                      std::to_string(fields_.size()) + " (";
    for (size_t i = 0; i < fields_.size(); ++i) msg += (i ? ", " : "") + fields_[i].name;
    return Status::error(msg + ")");
  }
  for (size_t i = 0; i < fields_.size(); ++i) {
    if (params[i].first != fields_[i].name)
      return Status::error("tiling param name mismatch at position " + std::to_string(i) + ": got '" + params[i].first +
                           "', expected '" + fields_[i].name + "'");
    const int64_t v = params[i].second;
    if (fields_[i].type == "int32" || fields_[i].type == "int32_t") {
      const int32_t w = static_cast<int32_t>(v);
      uint8_t buf[4];
      std::memcpy(buf, &w, 4);
      bytes.insert(bytes.end(), buf, buf + 4);
    } else {
      uint8_t buf[8];
      std::memcpy(buf, &v, 8);
      bytes.insert(bytes.end(), buf, buf + 8);
    }
  }
  return Status::success();
}

Status parseNamedTilingParams(const std::string &text, std::map<std::string, int64_t> &out) {
  out.clear();
  std::istringstream ss(text);
  std::string tok;
  while (std::getline(ss, tok, ',')) {
    size_t b = tok.find_first_not_of(" \t");
    if (b == std::string::npos) continue;
    tok = tok.substr(b, tok.find_last_not_of(" \t") - b + 1);
    const size_t eq = tok.find('=');
    if (eq == std::string::npos || eq == 0) return Status::error("invalid tiling token: " + tok);
    char *end = nullptr;
    const std::string val = tok.substr(eq + 1);
    const long long v = std::strtoll(val.c_str(), &end, 10);
    if (val.empty() || !end || *end != '\0') return Status::error("invalid tiling value: " + tok);
    out[tok.substr(0, eq)] = v;
  }
  return Status::success();
}

Status packTilingBytes(const TilingBinding &tiling, std::vector<uint8_t> &bytes) {
  bytes.clear();
  if (!tiling.present) return Status::success();
  if (!tiling.binaryPath.empty()) {
    if (Status s = readFileBytes(tiling.binaryPath, bytes); !s) return Status::error("cannot read tiling binary: " + tiling.binaryPath);
    return Status::success();
  }
  if (!tiling.schemaPath.empty()) {
    TilingSchema schema;
    if (Status s = TilingSchema::fromJsonFile(tiling.schemaPath, schema); !s) return s;
    std::map<std::string, int64_t> named;
    if (Status s = parseNamedTilingParams(tiling.params, named); !s) return s;
    std::vector<std::pair<std::string, int64_t>> ordered;
    for (const auto &f : schema.fields()) {
      auto it = named.find(f.name);
      if (it == named.end()) return Status::error("tiling params missing field: " + f.name);
      ordered.emplace_back(f.name, it->second);
    }
    return schema.pack(ordered, bytes);
  }
  if (!tiling.params.empty()) return Status::error("tiling params require either a schema path or a binary path");
  return Status::success();
}

} // namespace afir
