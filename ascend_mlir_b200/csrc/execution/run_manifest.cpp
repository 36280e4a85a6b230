#include "execution/run_manifest.h"

#include <sys/stat.h>

#include <sstream>

#include "common/json.h"

namespace afir {
namespace {

bool fileExists(const std::string &p) {
  struct stat st;
  return ::stat(p.c_str(), &st) == 0;
}

Status requireString(const json::Value &obj, const char *key, std::string &out) {
  const json::Value *v = obj.find(key);
  if (!v || !v->isString()) return Status::error(std::string("missing required string field: ") + key);
  out = v->asString();
  return Status::success();
}

Status parseBinding(const json::Value &obj, TensorBinding &b) {
  if (Status s = requireString(obj, "name", b.name); !s) return s;
  const std::string source = obj.getString("source", "external_file");
  if (source == "external_file") {
    b.sourceKind = BindingSourceKind::ExternalFile;
    b.path = obj.getString("path");
  } else if (source == "task_output") {
    b.sourceKind = BindingSourceKind::TaskOutput;
    if (Status s = requireString(obj, "upstream_task", b.upstreamTaskId); !s) return s;
    if (Status s = requireString(obj, "upstream_output", b.upstreamOutputName); !s) return s;
  } else {
    return Status::error("unsupported tensor binding source: " + source);
  }
  if (const json::Value *shape = obj.find("shape")) {
    if (!shape->isArray()) return Status::error("tensor binding shape must be an array");
    std::vector<int64_t> dims;
    for (const auto &d : shape->asArray()) {
      if (!d.isInt() || d.asInt() < 0) return Status::error("tensor binding shape entries must be non-negative integers");
      dims.push_back(d.asInt());
    }
    b.shape = dims;
  }
  if (const json::Value *dt = obj.find("dtype")) {
    NpyDType t;
    if (!dt->isString() || !parseNpyDTypeName(dt->asString(), t))
      return Status::error("unsupported tensor dtype: " + (dt->isString() ? dt->asString() : std::string("<non-string>")));
    b.dtype = t;
  }
  return Status::success();
}

Status parseBindings(const json::Value &root, const char *field, std::vector<TensorBinding> &out) {
  const json::Value *arr = root.find(field);
  if (!arr) return Status::success();
  if (!arr->isArray()) return Status::error(std::string(field) + " must be an array");
  for (const auto &v : arr->asArray()) {
    if (!v.isObject()) return Status::error(std::string(field) + " entries must be objects");
    TensorBinding b;
    if (Status s = parseBinding(v, b); !s) return s;
    out.push_back(std::move(b));
  }
  return Status::success();
}

Status parseTask(const json::Value &root, const std::string &defaultRoot, RuntimeTask &task) {
  if (Status s = requireString(root, "task_id", task.taskId); !s) return s;
  std::string artifactRoot = root.getString("artifact_root", defaultRoot);
  if (artifactRoot.empty()) return Status::error("missing required string field: artifact_root");
  task.artifact.artifactRoot = artifactRoot;
  if (const json::Value *deps = root.find("dependencies")) {
    if (!deps->isArray()) return Status::error("dependencies must be an array");
    for (const auto &d : deps->asArray()) {
      if (!d.isString()) return Status::error("dependencies entries must be strings");
      task.dependencies.push_back(d.asString());
    }
  }
  if (Status s = parseBindings(root, "inputs", task.invocation.inputs); !s) return s;
  if (Status s = parseBindings(root, "outputs", task.invocation.outputs); !s) return s;
  if (Status s = parseBindings(root, "expected_outputs", task.invocation.expectedOutputs); !s) return s;
  if (const json::Value *t = root.find("tiling")) {
    if (!t->isObject()) return Status::error("tiling must be an object");
    task.invocation.tiling.present = true;
    task.invocation.tiling.schemaPath = t->getString("schema");
    task.invocation.tiling.params = t->getString("params");
    task.invocation.tiling.binaryPath = t->getString("binary");
  }
  task.invocation.blockDim = static_cast<int>(root.getInt("block_dim", task.invocation.blockDim));
  task.invocation.workspaceSize = static_cast<size_t>(root.getInt("workspace_size", static_cast<int64_t>(task.invocation.workspaceSize)));
  task.invocation.enableProfiling = root.getBool("profiling", false);
  task.invocation.atol = root.getDouble("atol", task.invocation.atol);
  task.invocation.rtol = root.getDouble("rtol", task.invocation.rtol);
  return Status::success();
}

} // namespace

Status loadArtifactFromRoot(const std::string &root, KernelArtifact &out) {
  std::string manifest = root + "/out/manifest.txt";
  if (!fileExists(manifest)) manifest = root + "/manifest.txt";
  std::string text;
  if (Status s = readFileText(manifest, text); !s) return Status::error("artifact manifest not found under: " + root);
  out = KernelArtifact();
  out.artifactRoot = root;
  out.manifestPath = manifest;
  std::istringstream ss(text);
  std::string line;
  while (std::getline(ss, line)) {
    const size_t eq = line.find('=');
    if (eq == std::string::npos) continue;
    const std::string key = line.substr(0, eq), val = line.substr(eq + 1);
    if (key == "kernel_name") out.kernelName = val;
    else if (key == "soc_version") out.socVersion = val;
    else if (key == "kernel_kind") out.kernelKind = val == "cube" ? KernelKind::Cube : val == "mix" ? KernelKind::Mix : KernelKind::Vec;
    else if (key == "device_binary_path") out.deviceBinaryPath = val;
  }
  if (out.kernelName.empty()) return Status::error("artifact manifest has no kernel_name: " + manifest);
  if (out.deviceBinaryPath.empty()) return Status::error("artifact manifest has no device_binary_path: " + manifest);
  if (!fileExists(out.deviceBinaryPath)) {
    // artifact roots may have been moved: fall back to the binary next to the manifest
    const std::string sibling = manifest.substr(0, manifest.rfind('/')) + "/" + out.kernelName + ".bin";
    if (fileExists(sibling)) out.deviceBinaryPath = sibling;
    else return Status::error("device binary not found: " + out.deviceBinaryPath);
  }
  return Status::success();
}

Status loadRunManifest(const std::string &path, RunManifestSpec &out) {
  std::string text;
  if (Status s = readFileText(path, text); !s) return Status::error("cannot read run manifest: " + path);
  json::Value root;
  std::string err;
  if (!json::parse(text, root, err)) return Status::error("invalid JSON in run manifest: " + path);
  if (!root.isObject()) return Status::error("run manifest root must be an object: " + path);
  out = RunManifestSpec();
  if (Status s = requireString(root, "backend", out.backendName); !s) return s;
  if (out.backendName != "cuda" && out.backendName != "sim" && out.backendName != "npu")
    return Status::error("unsupported backend: " + out.backendName);
  const std::string defaultRoot = root.getString("artifact_root");
  if (const json::Value *tasks = root.find("tasks")) {
    if (!tasks->isArray()) return Status::error("tasks must be an array");
    for (const auto &t : tasks->asArray()) {
      if (!t.isObject()) return Status::error("tasks entries must be objects");
      RuntimeTask task;
      if (Status s = parseTask(t, defaultRoot, task); !s) return s;
      out.tasks.push_back(std::move(task));
    }
  } else {
    RuntimeTask task;
    if (Status s = parseTask(root, defaultRoot, task); !s) return s;
    out.tasks.push_back(std::move(task));
  }
  if (out.tasks.empty()) return Status::error("run manifest must contain at least one task");
  return Status::success();
}

Status buildTaskGraph(const RunManifestSpec &spec, TaskGraph &graph) {
  graph = TaskGraph();
  for (RuntimeTask task : spec.tasks) {
    if (Status s = loadArtifactFromRoot(task.artifact.artifactRoot, task.artifact); !s) return s;
    if (Status s = graph.addTask(task); !s) return s;
  }
  return Status::success();
}

} // namespace afir
