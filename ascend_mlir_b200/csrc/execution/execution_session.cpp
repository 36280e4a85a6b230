#include "execution/execution_session.h"

#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdlib>
#include <fstream>

#include "common/json.h"
#include "runtime/executor.h"

namespace afir {
namespace {

bool makeDirs(const std::string &path) {
  std::string cur;
  for (size_t i = 0; i <= path.size(); ++i) {
    if (i == path.size() || path[i] == '/') {
      if (!cur.empty() && ::mkdir(cur.c_str(), 0755) != 0 && errno != EEXIST) return false;
    }
    if (i < path.size()) cur.push_back(path[i]);
  }
  return true;
}

const char *kindName(KernelKind k) { return k == KernelKind::Cube ? "cube" : k == KernelKind::Mix ? "mix" : "vec"; }

json::Value tensorArray(const std::vector<TensorBinding> &bindings, const std::vector<NDArray> &arrays) {
  json::Array out;
  for (size_t i = 0; i < bindings.size() && i < arrays.size(); ++i) {
    json::Value t;
    t.set("name", bindings[i].name);
    t.set("path", bindings[i].path);
    json::Array shape;
    for (int64_t d : arrays[i].shape) shape.push_back(json::Value(d));
    t.set("shape", json::Value(std::move(shape)));
    t.set("dtype", npyDTypeName(arrays[i].dtype));
    out.push_back(std::move(t));
  }
  return json::Value(std::move(out));
}

class CudaBackendDriver final : public ExecutionBackendDriver {
public:
  explicit CudaBackendDriver(int device) : device_(device) {}

  Status run(const ExecutionRequest &request, ExecutionResult &result) override {
    const RuntimeTask &task = request.task;
    const ExecutionInvocation &inv = task.invocation;
    result = ExecutionResult();
    result.taskId = task.taskId;

    // ---- bindings ----
    std::vector<NDArray> inputs(inv.inputs.size());
    for (size_t i = 0; i < inv.inputs.size(); ++i)
      if (Status s = loadNpy(inv.inputs[i].path, inputs[i]); !s) return s.withStage("cuda:bindings");
    std::vector<NDArray> expected(inv.expectedOutputs.size());
    for (size_t i = 0; i < inv.expectedOutputs.size(); ++i)
      if (Status s = loadNpy(inv.expectedOutputs[i].path, expected[i]); !s) return s.withStage("cuda:bindings");
    if (inv.outputs.empty()) return Status::error("[cuda:bindings] task '" + task.taskId + "' declares no outputs");
    if (!expected.empty() && expected.size() != inv.outputs.size())
      return Status::error("[cuda:bindings] expected_outputs count differs from outputs");
    std::vector<NDArray> outputs(inv.outputs.size());
    for (size_t i = 0; i < inv.outputs.size(); ++i) {
      const TensorBinding &b = inv.outputs[i];
      if (b.shape && b.dtype) {
        outputs[i].shape = *b.shape;
        outputs[i].dtype = *b.dtype;
      } else if (i < expected.size()) {
        outputs[i].shape = expected[i].shape;
        outputs[i].dtype = expected[i].dtype;
      } else {
        return Status::error("[cuda:bindings] output '" + b.name + "' needs shape and dtype, or an expected output to take them from");
      }
      outputs[i].allocate();
    }
    std::vector<uint8_t> tiling;
    if (Status s = packTilingBytes(inv.tiling, tiling); !s) return s.withStage("cuda:bindings");

    // ---- artifact ----
    std::vector<uint8_t> binary;
    if (Status s = readFileBytes(task.artifact.deviceBinaryPath, binary); !s) return s.withStage("cuda:artifact");

    // ---- launch ----
    if (!executor_) {
      executor_ = std::make_unique<CudaExecutor>();
      if (Status s = executor_->initialize(device_); !s) return s.withStage("cuda:device");
    }
    std::vector<const void *> inPtrs;
    std::vector<size_t> inBytes;
    for (auto &a : inputs) { inPtrs.push_back(a.data()); inBytes.push_back(a.nbytes()); }
    std::vector<void *> outPtrs;
    std::vector<size_t> outBytes;
    for (auto &a : outputs) { outPtrs.push_back(a.data()); outBytes.push_back(a.nbytes()); }
    RunRequest req;
    req.binary = binary.data();
    req.binaryLen = binary.size();
    req.functionName = task.artifact.kernelName;
    req.numInputs = static_cast<int>(inputs.size());
    req.inputPtrs = inPtrs.data();
    req.inputBytes = inBytes.data();
    req.numOutputs = static_cast<int>(outputs.size());
    req.outputPtrs = outPtrs.data();
    req.outputBytes = outBytes.data();
    req.tiling = tiling.data();
    req.tilingLen = tiling.size();
    req.blockDim = inv.blockDim;
    req.magic = task.artifact.kernelKind == KernelKind::Cube ? kMagicCube : kMagicVec;
    const auto t0 = std::chrono::steady_clock::now();
    if (Status s = executor_->runHost(req); !s) return s;  // already stage-tagged
    const double wallUs = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();

    // ---- validate ----
    if (!expected.empty()) {
      if (Status s = compareRuntimeOutputs(outputs, expected, inv.atol, inv.rtol, result.comparison); !s)
        return s.withStage("cuda:validate");
      result.validated = true;
      if (!result.comparison.passed) return Status::error("[cuda:validate] " + result.comparison.errorMessage);
    }

    // ---- outputs ----
    for (size_t i = 0; i < outputs.size(); ++i) {
      if (inv.outputs[i].path.empty()) continue;
      if (Status s = saveNpy(inv.outputs[i].path, outputs[i]); !s) return s.withStage("cuda:write_outputs");
      result.producedFiles.push_back(inv.outputs[i].path);
    }

    // ---- profile ----
    result.profileTrace.sessionId = request.sessionId;
    result.profileTrace.counters["kernel_launches"] = executor_->lastLaunchCount();
    if (inv.enableProfiling) {
      double kernelUs = 0.0;
      if (Status s = executor_->profileResident(req, 20, kernelUs); !s) return s;
      const std::string dir = request.workingDirectory + "/opprof/cuda/" + task.taskId;
      if (!makeDirs(dir)) return Status::error("[cuda:profiling] cannot create profile directory: " + dir);
      const std::string path = dir + "/trace.json";
      json::Value root;
      root.set("schema_version", 1);
      root.set("backend", "cuda");
      root.set("session_id", request.sessionId);
      root.set("task_id", task.taskId);
      root.set("kernel_name", task.artifact.kernelName);
      root.set("kernel_kind", kindName(task.artifact.kernelKind));
      root.set("soc_version", task.artifact.socVersion);
      root.set("block_dim", inv.blockDim);
      root.set("workspace_size", static_cast<int64_t>(inv.workspaceSize));
      root.set("cycle_count", kernelUs);
      root.set("elapsed_us", kernelUs);
      root.set("score", kernelUs);
      root.set("end_to_end_us", wallUs);
      root.set("validation_passed", !result.validated || result.comparison.passed);
      root.set("artifact_root", task.artifact.artifactRoot);
      root.set("inputs", tensorArray(inv.inputs, inputs));
      root.set("outputs", tensorArray(inv.outputs, outputs));
      json::Value til;
      til.set("schema", inv.tiling.schemaPath);
      til.set("params", inv.tiling.params);
      til.set("binary", inv.tiling.binaryPath);
      til.set("bytes", static_cast<int64_t>(tiling.size()));
      root.set("tiling", std::move(til));
      std::ofstream os(path, std::ios::trunc);
      os << json::dump(root, 2) << "\n";
      if (!os) return Status::error("[cuda:profiling] cannot write profile artifact: " + path);
      ProfileEvent ev;
      ev.taskId = task.taskId;
      ev.backend = "cuda";
      ev.artifactPath = path;
      ev.score = kernelUs;
      result.profileTrace.events.push_back(ev);
    }
    return Status::success();
  }

private:
  int device_;
  std::unique_ptr<CudaExecutor> executor_;
};

} // namespace

std::shared_ptr<ExecutionBackendDriver> createCudaBackendDriver(int deviceId) {
  return std::make_shared<CudaBackendDriver>(deviceId);
}

std::pair<std::string, std::string> parseErrorStage(const std::string &message) {
  if (message.empty() || message[0] != '[') return {"", message};
  const size_t end = message.find(']');
  if (end == std::string::npos || end <= 1) return {"", message};
  const std::string prefix = message.substr(1, end - 1);
  const size_t split = prefix.find(':');
  if (split == std::string::npos || split + 1 >= prefix.size()) return {"", message};
  std::string rest = message.substr(end + 1);
  const size_t b = rest.find_first_not_of(" \t");
  rest = b == std::string::npos ? "" : rest.substr(b);
  return {prefix.substr(split + 1), rest};
}

ExecutionSession::ExecutionSession(std::string backendName, std::shared_ptr<ExecutionBackendDriver> driver)
    : backendName_(std::move(backendName)), driver_(std::move(driver)) {}

Status ExecutionSession::plan(const TaskGraph &graph, SessionPlan &plan) const {
  return graph.topologicalOrder(plan.orderedTaskIds);
}

SessionRunSummary ExecutionSession::run(const TaskGraph &graph, const std::string &workRoot) {
  SessionRunSummary summary;
  auto fail = [&](const std::string &message) {
    summary.success = false;
    summary.rawErrorMessage = message;
    auto parts = parseErrorStage(message);
    summary.errorStage = parts.first;
    summary.errorMessage = parts.second;
    return summary;
  };
  std::vector<RuntimeTask> order;
  if (Status s = graph.orderedTasks(order); !s) return fail(s.message());
  for (const auto &t : order)
    if (!t.invocation.expectedOutputs.empty()) summary.validationRan = true;

  std::string workDir = workRoot;
  if (workDir.empty()) {
    const char *tmp = std::getenv("TMPDIR");
    const std::string base = std::string(tmp && *tmp ? tmp : "/tmp") + "/afir-cuda-runtime";
    if (!makeDirs(base)) return fail("cannot create runtime session directory: " + base);
    std::string pattern = base + "/runtime-session-XXXXXX";
    std::vector<char> buf(pattern.begin(), pattern.end());
    buf.push_back('\0');
    if (!::mkdtemp(buf.data())) return fail("cannot create runtime session directory under: " + base);
    workDir = buf.data();
  } else if (!makeDirs(workDir)) {
    return fail("cannot create runtime session directory: " + workDir);
  }
  const std::string sessionId = workDir.substr(workDir.rfind('/') + 1);
  summary.profileTrace.sessionId = sessionId;
  summary.profileTrace.attributes["working_directory"] = workDir;
  summary.profileTrace.attributes["scheduler"] = "serial";
  summary.profileTrace.counters["planned_task_count"] = static_cast<int64_t>(order.size());
  if (!driver_) return fail("[cuda:device] no execution backend driver");

  std::map<std::string, std::map<std::string, std::string>> producedByTask;  // task -> output name -> file
  int64_t launched = 0;
  for (RuntimeTask task : order) {
    // resolve bindings: upstream task outputs become files, unnamed outputs get a file in the session directory
    for (TensorBinding &in : task.invocation.inputs) {
      if (in.sourceKind != BindingSourceKind::TaskOutput) continue;
      auto t = producedByTask.find(in.upstreamTaskId);
      if (t == producedByTask.end()) return fail("[cuda:bindings] input '" + in.name + "' refers to unknown upstream task '" + in.upstreamTaskId + "'");
      auto o = t->second.find(in.upstreamOutputName);
      if (o == t->second.end())
        return fail("[cuda:bindings] upstream task '" + in.upstreamTaskId + "' has no output '" + in.upstreamOutputName + "'");
      in.path = o->second;
    }
    for (TensorBinding &out : task.invocation.outputs)
      if (out.path.empty()) out.path = workDir + "/" + task.taskId + "." + out.name + ".npy";
    ExecutionRequest request;
    request.sessionId = sessionId;
    request.task = task;
    request.workingDirectory = workDir;
    ExecutionResult result;
    if (Status s = driver_->run(request, result); !s) {
      summary.results.push_back(std::move(result));
      summary.validationPassed = false;
      return fail(s.message());
    }
    for (const TensorBinding &out : task.invocation.outputs) producedByTask[task.taskId][out.name] = out.path;
    for (const ProfileEvent &ev : result.profileTrace.events) {
      summary.profileTrace.events.push_back(ev);
      summary.profileArtifactPaths.push_back(ev.artifactPath);
    }
    for (const auto &c : result.profileTrace.counters) summary.profileTrace.counters[c.first] += c.second;
    ++launched;
    summary.results.push_back(std::move(result));
  }
  summary.profileTrace.counters["serialized_launch_count"] = launched;
  summary.profileTrace.counters["max_in_flight_tasks"] = order.empty() ? 0 : 1;
  summary.validationPassed = summary.validationRan;
  summary.success = true;
  return summary;
}

} // namespace afir
