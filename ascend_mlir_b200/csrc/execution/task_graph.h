// Task graph of kernel runs: tasks, tensor bindings (files or upstream task outputs), tiling, validation
// settings, and a dependency-ordered plan (Kahn's algorithm; duplicate / empty / unknown / cyclic ids are
// errors).  Same shapes and defaults as the reference's include/Runtime/Execution/TaskGraph.h and
// lib/Runtime/Execution/TaskGraph.cpp:13-80, with "cuda" as the execution backend.
#pragma once

#include <cstdint>
#include <optional>
#include <string>
#include <vector>

#include "common/status.h"
#include "support/npy_io.h"
#include "support/tiling_schema.h"

namespace afir {

enum class KernelKind { Vec, Cube, Mix };
enum class BindingSourceKind { ExternalFile, TaskOutput };

struct KernelArtifact {
  std::string kernelName;
  KernelKind kernelKind = KernelKind::Vec;
  std::string socVersion;
  std::string artifactRoot;
  std::string deviceBinaryPath;
  std::string manifestPath;
};

struct TensorBinding {
  std::string name;
  BindingSourceKind sourceKind = BindingSourceKind::ExternalFile;
  std::string path;
  std::string upstreamTaskId;
  std::string upstreamOutputName;
  std::optional<std::vector<int64_t>> shape;
  std::optional<NpyDType> dtype;
};

struct ExecutionInvocation {
  std::vector<TensorBinding> inputs;
  std::vector<TensorBinding> outputs;
  std::vector<TensorBinding> expectedOutputs;
  TilingBinding tiling;
  int blockDim = 1;
  size_t workspaceSize = 8192;
  bool enableProfiling = false;
  double atol = 1.0;
  double rtol = 1e-2;
};

struct RuntimeTask {
  std::string taskId;
  KernelArtifact artifact;
  std::vector<std::string> dependencies;
  ExecutionInvocation invocation;
};

class TaskGraph {
public:
  Status addTask(const RuntimeTask &task);
  Status orderedTasks(std::vector<RuntimeTask> &order) const;
  Status topologicalOrder(std::vector<std::string> &ids) const;
  size_t size() const { return tasks_.size(); }

private:
  std::vector<RuntimeTask> tasks_;
};

} // namespace afir
