#include "execution/execution_session.h"

#include <cstring>

#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <fstream>
#include <mutex>
#include <thread>

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
  CudaBackendDriver(int device, size_t maxStreams) : device_(device), maxStreams_(std::max<size_t>(maxStreams, 1)) {}

  BackendCapabilities capabilities() const override {
    BackendCapabilities caps;
    caps.supportsConcurrentDispatch = true;
    caps.supportsConcurrentExecution = true;
    caps.requiresSerializedLaunch = false;
    caps.maxConcurrentTasks = maxStreams_;
    caps.maxConcurrentStreams = maxStreams_;
    return caps;
  }
  ExecutionBackendKind kind() const override { return ExecutionBackendKind::Cuda; }

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

    // A tiling given as schema + named params is packed in the KERNEL's field order when the schema is not the
    // kernel's own: a manifest written for the reference's kernel names that kernel's tile parameters (TB_M, Tb_N,
    // ...: loop tile sizes this target has no use for) beside the dims; the dims are taken by name, launch
    // parameters the manifest does not mention keep their defaults (0 = the library chooses), anything else is ignored.
    if (inv.tiling.present && inv.tiling.binaryPath.empty() && !inv.tiling.schemaPath.empty()) {
      LaunchDescriptor desc;
      if (Status s = parseDescriptorBinary(binary.data(), binary.size(), desc); !s) return s.withStage("cuda:artifact");
      TilingSchema schema;
      bool same = TilingSchema::fromJsonFile(inv.tiling.schemaPath, schema) && schema.fields().size() == desc.tiling.size();
      for (size_t i = 0; same && i < desc.tiling.size(); ++i) same = schema.fields()[i].name == desc.tiling[i].name;
      if (!same) {
        std::map<std::string, int64_t> named;
        if (Status s = parseNamedTilingParams(inv.tiling.params, named); !s) return s.withStage("cuda:bindings");
        tiling.clear();
        for (const TilingField &f : desc.tiling) {
          auto it = named.find(f.name);
          int64_t v = it == named.end() ? 0 : it->second;
          if (it == named.end() && f.name.compare(0, 7, "dim_arg") == 0) {
            // dim_arg<N>_<D> is extent D of kernel argument N (inputs, then outputs): a dimension the manifest's
            // schema does not carry (the reference's kernel derives an output's extents from its inputs') is read
            // off the tensor bound to that argument
            const size_t us = f.name.find('_', 7);
            char *end = nullptr;
            const long argIndex = us == std::string::npos ? -1 : std::strtol(f.name.c_str() + 7, &end, 10);
            const bool argOk = us != std::string::npos && end == f.name.c_str() + us && argIndex >= 0;
            const long dimIndex = argOk ? std::strtol(f.name.c_str() + us + 1, &end, 10) : -1;
            const bool dimOk = argOk && *end == '\0' && end != f.name.c_str() + us + 1 && dimIndex >= 0;
            const NDArray *bound = nullptr;
            if (dimOk && static_cast<size_t>(argIndex) < inputs.size()) bound = &inputs[argIndex];
            else if (dimOk && static_cast<size_t>(argIndex) < inputs.size() + outputs.size()) bound = &outputs[argIndex - inputs.size()];
            if (!bound || static_cast<size_t>(dimIndex) >= bound->shape.size())
              return Status::error("[cuda:bindings] tiling params missing field: " + f.name + " (a dimension of kernel '" + desc.kernel + "')");
            v = bound->shape[dimIndex];
          }
          uint8_t buf[8];
          if (f.bytes == 4) {
            const int32_t w = static_cast<int32_t>(v);
            std::memcpy(buf, &w, 4);
          } else {
            std::memcpy(buf, &v, 8);
          }
          tiling.insert(tiling.end(), buf, buf + f.bytes);
        }
      }
    }

    // ---- launch ----
    ExecutorLease executor_(*this);
    if (Status s = executor_.acquire(); !s) return s.withStage("cuda:device");
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
  // One executor (stream + buffer pool) per task in flight; idle ones are kept for the next task.
  class ExecutorLease {
  public:
    explicit ExecutorLease(CudaBackendDriver &owner) : owner_(owner) {}
    ~ExecutorLease() {
      if (!held_) return;
      std::lock_guard<std::mutex> lock(owner_.mutex_);
      owner_.idle_.push_back(std::move(held_));
    }
    Status acquire() {
      {
        std::lock_guard<std::mutex> lock(owner_.mutex_);
        if (!owner_.idle_.empty()) {
          held_ = std::move(owner_.idle_.back());
          owner_.idle_.pop_back();
          return Status::success();
        }
      }
      auto fresh = std::make_unique<CudaExecutor>();
      if (Status s = fresh->initialize(owner_.device_); !s) return s;
      held_ = std::move(fresh);
      return Status::success();
    }
    CudaExecutor *operator->() { return held_.get(); }

  private:
    CudaBackendDriver &owner_;
    std::unique_ptr<CudaExecutor> held_;
  };

  int device_;
  size_t maxStreams_;
  std::mutex mutex_;
  std::vector<std::unique_ptr<CudaExecutor>> idle_;
};

} // namespace

std::shared_ptr<ExecutionBackendDriver> createCudaBackendDriver(int deviceId, size_t maxStreams) {
  return std::make_shared<CudaBackendDriver>(deviceId, maxStreams);
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

// Everything the serial and the concurrent runners share.  `mutex` guards all of it in the concurrent case.
struct ExecutionSession::RunState {
  SessionRunSummary summary;
  std::vector<RuntimeTask> order;
  std::string workDir;
  std::string sessionId;
  std::map<std::string, std::map<std::string, std::string>> producedByTask;  // task -> output name -> file
  std::map<std::string, ExecutionResult> resultByTask;
  std::string firstError;
  std::mutex mutex;

  // Upstream task outputs become files; outputs without a path get one in the session directory.
  Status resolveBindings(RuntimeTask &task) const {
    for (TensorBinding &in : task.invocation.inputs) {
      if (in.sourceKind != BindingSourceKind::TaskOutput) continue;
      auto t = producedByTask.find(in.upstreamTaskId);
      if (t == producedByTask.end())
        return Status::error("[cuda:bindings] input '" + in.name + "' refers to unknown upstream task '" + in.upstreamTaskId + "'");
      auto o = t->second.find(in.upstreamOutputName);
      if (o == t->second.end())
        return Status::error("[cuda:bindings] upstream task '" + in.upstreamTaskId + "' has no output '" + in.upstreamOutputName + "'");
      in.path = o->second;
    }
    for (TensorBinding &out : task.invocation.outputs)
      if (out.path.empty()) out.path = workDir + "/" + task.taskId + "." + out.name + ".npy";
    return Status::success();
  }
  void recordSuccess(const RuntimeTask &task, ExecutionResult &&result) {
    for (const TensorBinding &out : task.invocation.outputs) producedByTask[task.taskId][out.name] = out.path;
    for (const auto &c : result.profileTrace.counters) summary.profileTrace.counters[c.first] += c.second;
    resultByTask[task.taskId] = std::move(result);
  }
  // Results, profile events and artifact paths in plan order, whatever order the tasks finished in.
  void collect() {
    for (const RuntimeTask &t : order) {
      auto it = resultByTask.find(t.taskId);
      if (it == resultByTask.end()) continue;
      for (const ProfileEvent &ev : it->second.profileTrace.events) {
        summary.profileTrace.events.push_back(ev);
        summary.profileArtifactPaths.push_back(ev.artifactPath);
      }
      summary.results.push_back(std::move(it->second));
    }
  }
};

static bool serialSchedulerForced() {
  for (const char *name : {"ASCEND_RUNTIME_FORCE_SERIAL_SCHEDULER", "AFIR_RUNTIME_FORCE_SERIAL_SCHEDULER"}) {
    const char *v = std::getenv(name);
    if (v && *v && std::string(v) != "0") return true;
  }
  return false;
}

void ExecutionSession::runSerial(RunState &st) {
  ProfileTrace &trace = st.summary.profileTrace;
  trace.attributes["scheduler"] = "serial";
  trace.attributes["scheduler_mode"] = "serial";
  int64_t launched = 0;
  for (RuntimeTask task : st.order) {
    if (Status s = st.resolveBindings(task); !s) {
      st.firstError = s.message();
      return;
    }
    ExecutionRequest request;
    request.sessionId = st.sessionId;
    request.task = task;
    request.workingDirectory = st.workDir;
    ExecutionResult result;
    if (Status s = driver_->run(request, result); !s) {
      st.resultByTask[task.taskId] = std::move(result);
      st.firstError = s.message();
      return;
    }
    st.recordSuccess(task, std::move(result));
    ++launched;
  }
  trace.counters["serialized_launch_count"] = launched;
  trace.counters["max_in_flight_tasks"] = st.order.empty() ? 0 : 1;
}

void ExecutionSession::runConcurrent(RunState &st, const TaskGraph &graph, const BackendCapabilities &caps) {
  GlobalScheduler &scheduler = scheduler_ ? *scheduler_ : globalScheduler();
  ProfileTrace &trace = st.summary.profileTrace;
  trace.attributes["scheduler"] = "concurrent";
  trace.attributes["scheduler_mode"] = "concurrent";
  trace.attributes["scheduler_scope"] = "global";

  SessionHandle handle;
  Status submitted = scheduling_ ? scheduler.submit(driver_->kind(), caps, graph, *scheduling_, handle)
                                 : scheduler.submit(driver_->kind(), caps, graph, handle);
  if (!submitted) {
    st.firstError = submitted.message();
    return;
  }
  const std::string globalId = handle.sessionId();
  int64_t roots = 0;
  for (const RuntimeTask &t : st.order) roots += t.dependencies.empty();
  trace.counters["frontier_count"] = 1;
  trace.counters["max_frontier_width"] = roots;

  size_t inFlight = 0, maxInFlight = 0;
  auto noteError = [&](const std::string &message) {  // st.mutex held
    if (st.firstError.empty()) st.firstError = message;
  };
  auto worker = [&]() {
    while (true) {
      std::optional<RuntimeTask> next;
      if (Status s = scheduler.waitAndAcquireTask(globalId, next); !s) {
        std::lock_guard<std::mutex> lock(st.mutex);
        noteError(s.message());
        return;
      }
      if (!next) return;  // drained: all done, or failed and nothing of ours still runs
      RuntimeTask task = std::move(*next);
      Status ready;
      {
        std::lock_guard<std::mutex> lock(st.mutex);
        ready = st.resolveBindings(task);
        if (ready) maxInFlight = std::max(maxInFlight, ++inFlight);
        else noteError(ready.message());
      }
      if (!ready) {
        scheduler.failTask(globalId, task.taskId);
        continue;
      }
      ExecutionRequest request;
      request.sessionId = st.sessionId;
      request.task = task;
      request.workingDirectory = st.workDir;
      ExecutionResult result;
      const Status ran = driver_->run(request, result);
      {
        std::lock_guard<std::mutex> lock(st.mutex);
        --inFlight;
        if (ran) st.recordSuccess(task, std::move(result));
        else {
          st.resultByTask[task.taskId] = std::move(result);
          noteError(ran.message());
        }
      }
      if (!ran) {
        if (Status s = scheduler.failTask(globalId, task.taskId); !s) {
          std::lock_guard<std::mutex> lock(st.mutex);
          noteError(s.message());
        }
        continue;
      }
      size_t newlyReady = 0;
      const Status done = scheduler.completeTask(globalId, task.taskId, &newlyReady);
      std::lock_guard<std::mutex> lock(st.mutex);
      if (!done) noteError(done.message());
      else if (newlyReady > 0) {
        trace.counters["frontier_count"] += static_cast<int64_t>(newlyReady);
        trace.counters["max_frontier_width"] = std::max(trace.counters["max_frontier_width"], static_cast<int64_t>(newlyReady));
      }
    }
  };

  const size_t hardware = std::thread::hardware_concurrency() ? std::thread::hardware_concurrency() : 4;
  const size_t workers = std::max<size_t>(1, std::min({st.order.size(), std::max<size_t>(caps.maxConcurrentTasks, 1), hardware}));
  std::vector<std::thread> pool;
  for (size_t i = 0; i < workers; ++i) pool.emplace_back(worker);
  for (std::thread &t : pool) t.join();

  const SchedulerObservabilitySnapshot snapshot = scheduler.observabilitySnapshot();
  scheduler.releaseSession(globalId);
  for (const auto &a : snapshot.attributes) trace.attributes[a.first] = a.second;
  for (const auto &c : snapshot.counters) trace.counters[c.first] = c.second;
  trace.counters["max_in_flight_tasks"] = static_cast<int64_t>(maxInFlight);
  trace.counters["worker_count"] = static_cast<int64_t>(workers);
  if (st.firstError.empty() && st.producedByTask.size() != st.order.size())
    st.firstError = "scheduler terminated with " + std::to_string(st.producedByTask.size()) + "/" +
                    std::to_string(st.order.size()) + " tasks completed";
}

SessionRunSummary ExecutionSession::run(const TaskGraph &graph, const std::string &workRoot) {
  RunState st;
  SessionRunSummary &summary = st.summary;
  auto fail = [&](const std::string &message) {
    summary.success = false;
    summary.validationPassed = false;
    summary.rawErrorMessage = message;
    auto parts = parseErrorStage(message);
    summary.errorStage = parts.first;
    summary.errorMessage = parts.second;
    return std::move(summary);
  };
  if (Status s = graph.orderedTasks(st.order); !s) return fail(s.message());
  for (const auto &t : st.order)
    if (!t.invocation.expectedOutputs.empty()) summary.validationRan = true;

  st.workDir = workRoot;
  if (st.workDir.empty()) {
    const char *tmp = std::getenv("TMPDIR");
    const std::string base = std::string(tmp && *tmp ? tmp : "/tmp") + "/afir-cuda-runtime";
    if (!makeDirs(base)) return fail("cannot create runtime session directory: " + base);
    std::string pattern = base + "/runtime-session-XXXXXX";
    std::vector<char> buf(pattern.begin(), pattern.end());
    buf.push_back('\0');
    if (!::mkdtemp(buf.data())) return fail("cannot create runtime session directory under: " + base);
    st.workDir = buf.data();
  } else if (!makeDirs(st.workDir)) {
    return fail("cannot create runtime session directory: " + st.workDir);
  }
  st.sessionId = st.workDir.substr(st.workDir.rfind('/') + 1);
  summary.profileTrace.sessionId = st.sessionId;
  summary.profileTrace.attributes["working_directory"] = st.workDir;
  summary.profileTrace.counters["planned_task_count"] = static_cast<int64_t>(st.order.size());
  if (!driver_) return fail("[cuda:device] no execution backend driver");

  const BackendCapabilities caps = driver_->capabilities();
  if (st.order.size() > 1 && caps.supportsConcurrentDispatch && !serialSchedulerForced()) runConcurrent(st, graph, caps);
  else runSerial(st);
  st.collect();
  if (!st.firstError.empty()) return fail(st.firstError);
  summary.validationPassed = summary.validationRan;
  summary.success = true;
  return std::move(summary);
}

} // namespace afir
