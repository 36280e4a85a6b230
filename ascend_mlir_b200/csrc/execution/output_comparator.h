// Output validation rule of the reference (lib/Runtime/Execution/OutputComparator.cpp:75-140): structural
// mismatches are errors; element i fails when |actual - expected| > atol + rtol * |expected| (in double, from
// the f32 value of either dtype); max and mean absolute difference are reported.
#pragma once

#include <string>
#include <vector>

#include "common/status.h"
#include "support/npy_io.h"

namespace afir {

struct OutputComparisonResult {
  bool passed = false;
  double maxAbsDiff = 0.0;
  double meanAbsDiff = 0.0;
  std::string errorMessage;
};

Status compareRuntimeOutputs(const std::vector<NDArray> &actual, const std::vector<NDArray> &expected, double atol,
                             double rtol, OutputComparisonResult &result);

// Element `idx` of a tensor as float (f16/bf16 widened exactly, integers converted).
float elementAsFloat(const NDArray &a, size_t idx);

} // namespace afir
