#include "execution/output_comparator.h"

#include <cmath>
#include <cstdio>
#include <cstring>

namespace afir {

float elementAsFloat(const NDArray &a, size_t idx) {
  const uint8_t *base = a.bytes.data();
  switch (a.dtype) {
  case NpyDType::F16: {
    uint16_t h;
    std::memcpy(&h, base + idx * 2, 2);
    const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu, frac = h & 0x3ffu;
    if (exp == 0) {  // zero or subnormal: value = frac * 2^-24
      const float v = static_cast<float>(frac) * 5.9604644775390625e-08f;
      return sign ? -v : v;
    }
    const uint32_t bits = exp == 31 ? (sign | 0x7f800000u | (frac << 13)) : (sign | ((exp + 112u) << 23) | (frac << 13));
    float r;
    std::memcpy(&r, &bits, 4);
    return r;
  }
  case NpyDType::BF16: {
    uint16_t h;
    std::memcpy(&h, base + idx * 2, 2);
    const uint32_t bits = static_cast<uint32_t>(h) << 16;
    float r;
    std::memcpy(&r, &bits, 4);
    return r;
  }
  case NpyDType::F32: {
    float v;
    std::memcpy(&v, base + idx * 4, 4);
    return v;
  }
  case NpyDType::INT8: return static_cast<float>(static_cast<int8_t>(base[idx]));
  case NpyDType::INT32: {
    int32_t v;
    std::memcpy(&v, base + idx * 4, 4);
    return static_cast<float>(v);
  }
  case NpyDType::INT64: {
    int64_t v;
    std::memcpy(&v, base + idx * 8, 8);
    return static_cast<float>(v);
  }
  case NpyDType::INT16: {
    int16_t v;
    std::memcpy(&v, base + idx * 2, 2);
    return static_cast<float>(v);
  }
  }
  return 0.0f;
}

Status compareRuntimeOutputs(const std::vector<NDArray> &actual, const std::vector<NDArray> &expected, double atol,
                             double rtol, OutputComparisonResult &result) {
  result = OutputComparisonResult();
  if (actual.size() != expected.size())
    return Status::error("output count mismatch: got " + std::to_string(actual.size()) + ", expected " +
                         std::to_string(expected.size()));
  result.passed = true;
  double total = 0.0;
  size_t elements = 0;
  for (size_t o = 0; o < actual.size(); ++o) {
    const NDArray &a = actual[o], &e = expected[o];
    const std::string tag = "output " + std::to_string(o);
    if (a.shape != e.shape) return Status::error(tag + " shape mismatch");
    if (a.dtype != e.dtype) return Status::error(tag + " dtype mismatch");
    if (a.nbytes() != e.nbytes()) return Status::error(tag + " byte-size mismatch");
    if (a.bytes.size() < a.nbytes() || e.bytes.size() < e.nbytes()) return Status::error(tag + " has null data pointer");
    const size_t n = a.numElements();
    elements += n;
    for (size_t i = 0; i < n; ++i) {
      const double av = elementAsFloat(a, i), ev = elementAsFloat(e, i);
      const double diff = std::fabs(av - ev);
      total += diff;
      if (diff > result.maxAbsDiff) result.maxAbsDiff = diff;
      if (!(diff <= atol + rtol * std::fabs(ev))) result.passed = false;
    }
  }
  result.meanAbsDiff = elements ? total / static_cast<double>(elements) : 0.0;
  if (!result.passed) {
    char buf[160];
    std::snprintf(buf, sizeof(buf), "output comparison failed: max_abs_diff=%g, mean_abs_diff=%g", result.maxAbsDiff,
                  result.meanAbsDiff);
    result.errorMessage = buf;
  }
  return Status::success();
}

} // namespace afir
