// TilingSchema / packTilingBytes: named tiling parameters -> the packed little-endian TilingData bytes
// a kernel takes.  Contract of the reference's lib/Runtime/Support/TilingSchema.cpp:13-100 and
// TilingPack.cpp:43-89: only 'name' and 'type' of tiling_params[] matter, schema order is byte order,
// names are checked position by position; bytes come from a binary file, else from schema + "k=v,..." text.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "common/json.h"
#include "common/status.h"

namespace afir {

struct TilingSchemaField {
  std::string name;
  std::string type = "int64";
};

class TilingSchema {
public:
  static Status fromJsonFile(const std::string &path, TilingSchema &out);
  static Status fromJsonValue(const json::Value &root, const std::string &origin, TilingSchema &out);
  const std::vector<TilingSchemaField> &fields() const { return fields_; }
  Status pack(const std::vector<std::pair<std::string, int64_t>> &params, std::vector<uint8_t> &bytes) const;

private:
  std::vector<TilingSchemaField> fields_;
};

struct TilingBinding {
  std::string schemaPath;
  std::string params;      // "TB_M=64,dim_arg0_0=640,..."
  std::string binaryPath;
  bool present = false;
};

Status parseNamedTilingParams(const std::string &text, std::map<std::string, int64_t> &out);
Status packTilingBytes(const TilingBinding &tiling, std::vector<uint8_t> &bytes);
Status readFileBytes(const std::string &path, std::vector<uint8_t> &out);
Status readFileText(const std::string &path, std::string &out);

} // namespace afir
