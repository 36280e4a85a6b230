// Execution session: plans a task graph, runs its tasks in dependency order through a backend driver,
// validates outputs against expected tensors, saves outputs as .npy and writes a profile trace per task.
// The driver is the test seam the reference uses (include/Runtime/Execution/ExecutionBackend.h:28-37):
// inject one and no device code runs.  The default driver executes on a CUDA device through CudaExecutor.
// Error messages carry the reference's stage tags, with "cuda" as the backend:
// [cuda:bindings|artifact|kernel_launch|validate|write_outputs|profiling].
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "execution/global_scheduler.h"
#include "execution/output_comparator.h"
#include "execution/task_graph.h"

namespace afir {

struct ProfileEvent {
  std::string taskId;
  std::string backend;
  std::string artifactPath;   // trace.json of the task
  double score = 0.0;         // median kernel microseconds (lower is better)
};

struct ProfileTrace {
  std::string sessionId;
  std::vector<ProfileEvent> events;
  std::map<std::string, std::string> attributes;
  std::map<std::string, int64_t> counters;
};

struct ExecutionRequest {
  std::string sessionId;
  RuntimeTask task;  // bindings already resolved to files
  std::string workingDirectory;
};

struct ExecutionResult {
  std::string taskId;
  std::vector<std::string> producedFiles;
  bool validated = false;
  OutputComparisonResult comparison;
  ProfileTrace profileTrace;
};

class ExecutionBackendDriver {
public:
  virtual ~ExecutionBackendDriver() = default;
  virtual Status run(const ExecutionRequest &request, ExecutionResult &result) = 0;
  // What the scheduler may assume.  The default is a driver that runs one task at a time; a driver that
  // reports supportsConcurrentDispatch must accept run() from several threads at once.
  virtual BackendCapabilities capabilities() const { return BackendCapabilities(); }
  virtual ExecutionBackendKind kind() const { return ExecutionBackendKind::Host; }
};

// Runs tasks on CUDA device `deviceId` (AFIR_CUDA_DEVICE, default 0).  Tasks dispatched at the same time
// each get an executor of their own (own stream, own pooled buffers), up to `maxStreams` of them.
std::shared_ptr<ExecutionBackendDriver> createCudaBackendDriver(int deviceId, size_t maxStreams = 4);

struct SessionPlan {
  std::vector<std::string> orderedTaskIds;
};

struct SessionRunSummary {
  bool success = false;
  bool validationRan = false;
  bool validationPassed = false;
  std::string errorStage;
  std::string errorMessage;     // without the stage tag
  std::string rawErrorMessage;  // as raised
  ProfileTrace profileTrace;
  std::vector<std::string> profileArtifactPaths;
  std::vector<ExecutionResult> results;
};

class ExecutionSession {
public:
  ExecutionSession(std::string backendName, std::shared_ptr<ExecutionBackendDriver> driver);
  Status plan(const TaskGraph &graph, SessionPlan &plan) const;
  // Never throws or returns an error: failures are reported in the summary.
  SessionRunSummary run(const TaskGraph &graph, const std::string &workRoot = "");
  const std::string &backendName() const { return backendName_; }
  // Graphs of more than one task go through a GlobalScheduler (the process-wide one unless another is set
  // here) when the driver supports concurrent dispatch and ASCEND_RUNTIME_FORCE_SERIAL_SCHEDULER /
  // AFIR_RUNTIME_FORCE_SERIAL_SCHEDULER is not set to a non-zero value: independent tasks then run on
  // worker threads, and the first failure cancels what has not started.
  void setScheduler(GlobalScheduler *scheduler) { scheduler_ = scheduler; }
  void setScheduling(const SessionSchedulingOptions &options) { scheduling_ = options; }

private:
  struct RunState;
  void runSerial(RunState &state);
  void runConcurrent(RunState &state, const TaskGraph &graph, const BackendCapabilities &caps);

  std::string backendName_;
  std::shared_ptr<ExecutionBackendDriver> driver_;
  GlobalScheduler *scheduler_ = nullptr;
  std::optional<SessionSchedulingOptions> scheduling_;
};

// "[cuda:validate] text" -> {"validate", "text"}; untagged messages give an empty stage.
std::pair<std::string, std::string> parseErrorStage(const std::string &message);

} // namespace afir
