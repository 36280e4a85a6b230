#include "support/npy_io.h"

#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <fstream>

namespace afir {

const char *npyDTypeName(NpyDType t) {
  switch (t) {
  case NpyDType::F16: return "f16";
  case NpyDType::BF16: return "bf16";
  case NpyDType::F32: return "f32";
  case NpyDType::INT8: return "i8";
  case NpyDType::INT32: return "i32";
  case NpyDType::INT64: return "i64";
  case NpyDType::INT16: return "i16";
  }
  return "?";
}

bool parseNpyDTypeName(const std::string &s, NpyDType &out) {
  if (s == "f16" || s == "float16") out = NpyDType::F16;
  else if (s == "bf16" || s == "bfloat16") out = NpyDType::BF16;
  else if (s == "f32" || s == "float32") out = NpyDType::F32;
  else if (s == "i8" || s == "int8") out = NpyDType::INT8;
  else if (s == "i32" || s == "int32") out = NpyDType::INT32;
  else if (s == "i64" || s == "int64") out = NpyDType::INT64;
  else if (s == "i16" || s == "int16") out = NpyDType::INT16;
  else return false;
  return true;
}

size_t npyDTypeBytes(NpyDType t) {
  switch (t) {
  case NpyDType::F16: case NpyDType::BF16: case NpyDType::INT16: return 2;
  case NpyDType::F32: case NpyDType::INT32: return 4;
  case NpyDType::INT8: return 1;
  case NpyDType::INT64: return 8;
  }
  return 0;
}

namespace {

// Value of a "'key': " entry of the header dict; empty when absent.
std::string headerField(const std::string &header, const std::string &key) {
  const std::string needle = "'" + key + "'";
  size_t p = header.find(needle);
  if (p == std::string::npos) return "";
  p = header.find(':', p + needle.size());
  if (p == std::string::npos) return "";
  ++p;
  while (p < header.size() && (header[p] == ' ' || header[p] == '\t')) ++p;
  if (p >= header.size()) return "";
  if (header[p] == '\'') {
    size_t e = header.find('\'', p + 1);
    return e == std::string::npos ? "" : header.substr(p + 1, e - p - 1);
  }
  if (header[p] == '(') {
    size_t e = header.find(')', p);
    return e == std::string::npos ? "" : header.substr(p, e - p + 1);
  }
  size_t e = p;
  while (e < header.size() && header[e] != ',' && header[e] != '}') ++e;
  return header.substr(p, e - p);
}

} // namespace

Status loadNpy(const std::string &path, NDArray &out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return Status::error("Cannot open: " + path);
  char magic[6] = {0};
  f.read(magic, 6);
  if (f.gcount() != 6 || std::memcmp(magic, "\x93NUMPY", 6) != 0) return Status::error("Not a .npy file: " + path);
  uint8_t ver[2] = {0, 0};
  f.read(reinterpret_cast<char *>(ver), 2);
  uint32_t hlen = 0;
  if (ver[0] == 1) {
    uint8_t b[2];
    f.read(reinterpret_cast<char *>(b), 2);
    hlen = static_cast<uint32_t>(b[0]) | (static_cast<uint32_t>(b[1]) << 8);
  } else {
    uint8_t b[4];
    f.read(reinterpret_cast<char *>(b), 4);
    hlen = static_cast<uint32_t>(b[0]) | (static_cast<uint32_t>(b[1]) << 8) | (static_cast<uint32_t>(b[2]) << 16) |
           (static_cast<uint32_t>(b[3]) << 24);
  }
  if (!f || hlen == 0 || hlen > (1u << 20)) return Status::error("Cannot parse header: " + path);
  std::string header(hlen, '\0');
  f.read(header.data(), hlen);
  if (static_cast<uint32_t>(f.gcount()) != hlen) return Status::error("Cannot parse header: " + path);

  const std::string shape = headerField(header, "shape");
  if (shape.size() < 2 || shape.front() != '(') return Status::error("Cannot parse shape: " + path);
  out = NDArray();
  {
    std::string tok;
    for (size_t i = 1; i < shape.size(); ++i) {
      const char c = shape[i];
      if (c >= '0' && c <= '9') tok.push_back(c);
      else if (c == ',' || c == ')') {
        if (!tok.empty()) out.shape.push_back(std::stoll(tok));
        tok.clear();
      } else if (c != ' ' && c != '\t') return Status::error("Cannot parse shape: " + path);
    }
  }
  const std::string descr = headerField(header, "descr");
  if (descr.empty()) return Status::error("Cannot parse dtype: " + path);
  if (descr == "<f2" || descr == "=f2") out.dtype = NpyDType::F16;
  else if (descr == "<V2" || descr == "=V2" || descr == "|V2" || descr == "<u2") out.dtype = NpyDType::BF16;
  else if (descr == "<f4" || descr == "=f4") out.dtype = NpyDType::F32;
  else if (descr == "<i1" || descr == "=i1" || descr == "|i1") out.dtype = NpyDType::INT8;
  else if (descr == "<i4" || descr == "=i4") out.dtype = NpyDType::INT32;
  else if (descr == "<i8" || descr == "=i8") out.dtype = NpyDType::INT64;
  else if (descr == "<i2" || descr == "=i2") out.dtype = NpyDType::INT16;
  else return Status::error("Unsupported dtype '" + descr + "': " + path);
  const bool fortran = headerField(header, "fortran_order").find("True") != std::string::npos;
  // The header's shape is checked against what the file holds before anything of that size is allocated (a damaged
  // header can claim terabytes).
  {
    const std::streampos dataBegin = f.tellg();
    f.seekg(0, std::ios::end);
    const std::streampos fileEnd = f.tellg();
    f.seekg(dataBegin);
    const unsigned long long available = fileEnd >= dataBegin ? static_cast<unsigned long long>(fileEnd - dataBegin) : 0ull;
    unsigned long long claimed = npyDTypeBytes(out.dtype);
    for (int64_t d : out.shape) {
      if (d != 0 && claimed > available / static_cast<unsigned long long>(d)) return Status::error("Truncated data in: " + path);
      claimed *= static_cast<unsigned long long>(d);
    }
  }
  out.allocate();
  f.read(reinterpret_cast<char *>(out.bytes.data()), static_cast<std::streamsize>(out.bytes.size()));
  if (static_cast<size_t>(f.gcount()) != out.bytes.size()) return Status::error("Truncated data in: " + path);
  // A column-major file (numpy writes one for, e.g., the result of indexing columns with an index array: the
  // reference's gather example saves its expected output that way) is brought into row-major order, which is what
  // every consumer of an NDArray assumes.  The reference's reader takes the bytes as they come
  // (lib/Runtime/Support/NpyIO.cpp:17-120 never looks at fortran_order) and so compares against permuted data.
  if (fortran && out.shape.size() > 1 && out.numElements() > 1) {
    const size_t eb = npyDTypeBytes(out.dtype), rank = out.shape.size();
    std::vector<uint8_t> rowMajor(out.bytes.size());
    std::vector<size_t> columnStride(rank, 1);  // element stride of every dim in the file's order
    for (size_t d = 1; d < rank; ++d) columnStride[d] = columnStride[d - 1] * static_cast<size_t>(out.shape[d - 1]);
    std::vector<int64_t> index(rank, 0);
    size_t from = 0;  // offset of `index` in the file's order, kept up to date while the row-major index advances
    for (size_t to = 0, n = out.numElements(); to < n; ++to) {
      std::memcpy(rowMajor.data() + to * eb, out.bytes.data() + from * eb, eb);
      for (size_t d = rank; d-- > 0;) {
        from += columnStride[d];
        if (++index[d] < out.shape[d]) break;
        from -= columnStride[d] * static_cast<size_t>(out.shape[d]);
        index[d] = 0;
      }
    }
    out.bytes.swap(rowMajor);
  }
  return Status::success();
}

Status saveNpy(const std::string &path, const NDArray &arr) {
  const char *descr = "<f4";
  switch (arr.dtype) {
  case NpyDType::F16: descr = "<f2"; break;
  case NpyDType::BF16: descr = "<V2"; break;
  case NpyDType::F32: descr = "<f4"; break;
  case NpyDType::INT8: descr = "|i1"; break;
  case NpyDType::INT32: descr = "<i4"; break;
  case NpyDType::INT16: descr = "<i2"; break;
  case NpyDType::INT64: descr = "<i8"; break;
  }
  std::string shape = "(";
  for (size_t i = 0; i < arr.shape.size(); ++i) {
    shape += std::to_string(arr.shape[i]);
    if (arr.shape.size() == 1 || i + 1 < arr.shape.size()) shape += ",";
  }
  shape += ")";
  std::string dict = std::string("{'descr': '") + descr + "', 'fortran_order': False, 'shape': " + shape + ", }";
  const size_t total = 10 + dict.size() + 1;  // magic + version + header length, dict, newline
  dict.append((64 - total % 64) % 64, ' ');
  dict.push_back('\n');
  if (dict.size() > 0xffff) return Status::error("Cannot write: header too long for " + path);

  std::string tmp = path + ".XXXXXX.tmp";
  {
    // unique sibling name: the final rename is atomic on one filesystem
    std::vector<char> pattern(path.begin(), path.end());
    const char *suffix = ".XXXXXX";
    pattern.insert(pattern.end(), suffix, suffix + 7);
    pattern.push_back('\0');
    int fd = ::mkstemp(pattern.data());
    if (fd < 0) return Status::error("Cannot create temp npy file for: " + path);
    ::close(fd);
    tmp.assign(pattern.data());
  }
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    if (!f) return Status::error("Cannot write: " + tmp);
    const uint16_t hlen = static_cast<uint16_t>(dict.size());
    const uint8_t prefix[4] = {1, 0, static_cast<uint8_t>(hlen & 0xff), static_cast<uint8_t>(hlen >> 8)};
    f.write("\x93NUMPY", 6);
    f.write(reinterpret_cast<const char *>(prefix), 4);
    f.write(dict.data(), static_cast<std::streamsize>(dict.size()));
    f.write(reinterpret_cast<const char *>(arr.bytes.data()), static_cast<std::streamsize>(arr.nbytes()));
    f.close();
    if (!f) {
      std::remove(tmp.c_str());
      return Status::error("Cannot finalize temp npy file: " + tmp);
    }
  }
  if (std::rename(tmp.c_str(), path.c_str()) != 0) {
    std::remove(tmp.c_str());
    return Status::error("Cannot replace npy output: " + path);
  }
  return Status::success();
}

} // namespace afir
