// .npy tensors for the runtime tools: version 1/2/3 files read, version 1 written (64-byte padded
// header, bf16 stored as '<V2' the way numpy writes void2), output replaced atomically (temp + rename).
// Same dtype set and error wording as the reference's lib/Runtime/Support/NpyIO.cpp:17-166.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "common/status.h"
#include "runtime/descriptor.h"

namespace afir {

enum class NpyDType { F16, BF16, F32, INT8, INT32, INT64, INT16 };
const char *npyDTypeName(NpyDType t);       // "f16", "bf16", ...
bool parseNpyDTypeName(const std::string &s, NpyDType &out);
size_t npyDTypeBytes(NpyDType t);

struct NDArray {
  NpyDType dtype = NpyDType::F32;
  std::vector<int64_t> shape;
  std::vector<uint8_t> bytes;

  size_t numElements() const {
    size_t n = 1;
    for (int64_t d : shape) n *= static_cast<size_t>(d);
    return n;
  }
  size_t nbytes() const { return numElements() * npyDTypeBytes(dtype); }
  void allocate() { bytes.assign(nbytes(), 0); }
  const void *data() const { return bytes.data(); }
  void *data() { return bytes.data(); }
};

Status loadNpy(const std::string &path, NDArray &out);
Status saveNpy(const std::string &path, const NDArray &arr);

} // namespace afir
