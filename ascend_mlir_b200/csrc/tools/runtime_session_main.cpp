// runtime-session: plan and run a task graph of kernel launches on the CUDA backend.
// Same command line, stdout/stderr key=value lines and exit codes (0 ok, 2 plan/run failure, 4 usage or
// preparation failure) as the reference's tools/runtime-session/runtime_session_main.cpp:30-110,244-397.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>

#include "execution/artifact_compiler.h"
#include "execution/execution_session.h"
#include "execution/profile_retention.h"
#include "execution/run_manifest.h"
#include "tools/cli_args.h"

using namespace afir;

namespace {

// Testing-only driver: reports success without touching a device (the reference exposes the same seam as
// --testing-driver npu-success).
class SuccessfulTestingDriver final : public ExecutionBackendDriver {
public:
  Status run(const ExecutionRequest &request, ExecutionResult &result) override {
    result = ExecutionResult();
    result.taskId = request.task.taskId;
    for (const TensorBinding &b : request.task.invocation.outputs) result.producedFiles.push_back(b.path);
    ProfileEvent ev;
    ev.taskId = request.task.taskId;
    ev.backend = "cuda";
    ev.artifactPath = request.workingDirectory + "/" + request.task.taskId + ".cuda-profile.json";
    ev.score = 1.0;
    {  // a minimal artifact, so that retention has something to keep
      std::ofstream os(ev.artifactPath, std::ios::trunc);
      os << "{\"schema_version\": 1, \"backend\": \"cuda\", \"task_id\": \"" << request.task.taskId
         << "\", \"score\": 1, \"cycle_count\": 1}\n";
      if (!os) return Status::error("[cuda:profiling] cannot write profile artifact: " + ev.artifactPath);
    }
    result.profileTrace.sessionId = request.sessionId;
    result.profileTrace.events.push_back(ev);
    return Status::success();
  }
};

void usage() {
  std::cout << "OVERVIEW: task graph runtime planning and execution CLI for artifacts and session graphs\n\n"
               "USAGE: runtime-session [options]\n\nOPTIONS:\n"
               "  --artifact-root=<dir>   Use an existing artifact root with a real manifest\n"
               "  --kernel=<file>         Kernel source (launch descriptor) to compile into a runtime artifact\n"
               "  --name=<string>         Kernel name override when compiling a new artifact\n"
               "  --output=<dir>          Artifact output directory when compiling\n"
               "  --soc=<string>          Target SoC version when compiling a new artifact\n"
               "  --kernel-kind=<string>  Kernel kind when compiling: vec, cube, or mix\n"
               "  --task-id=<string>      Task id to register in the task graph\n"
               "  --run-manifest=<file>   JSON manifest describing artifact root, bindings, and execution settings\n"
               "  --run                   Execute the prepared task graph runtime session\n";
}

// `asked`: the backend name of the manifest.  The reference's names "sim" and "npu" are accepted for this backend, and
// session.backend repeats the name that was asked for (its example scripts look for the line session.backend=sim);
// session.device_backend says what ran.
void printBackend(std::ostream &os, const ExecutionSession &session, const std::string &asked) {
  os << "session.backend=" << (asked.empty() ? session.backendName() : asked) << "\n";
  if (!asked.empty() && asked != session.backendName()) os << "session.device_backend=" << session.backendName() << "\n";
}

void printRunError(const ExecutionSession &session, const std::string &asked, const SessionRunSummary &summary) {
  printBackend(std::cerr, session, asked);
  std::cerr << "session.result=error\n";
  if (summary.validationRan && summary.errorStage == "validate") std::cerr << "session.validation=fail\n";
  if (!summary.errorStage.empty()) std::cerr << "session.error_stage=" << summary.errorStage << "\n";
  std::cerr << "session.error=" << summary.errorMessage << "\n";
  std::cerr << "Error: " << summary.rawErrorMessage << "\n";
}

} // namespace

int main(int argc, char **argv) {
  CliArgs args({"artifact-root", "kernel", "name", "output", "soc", "kernel-kind", "task-id", "run-manifest", "testing-driver",
                "cann-mlir", "npy-dir"},
               {"run"});
  std::string err;
  if (!args.parse(argc, argv, err)) {
    std::cerr << "runtime-session: " << err << "\n";
    return 1;
  }
  if (args.help()) { usage(); return 0; }

  std::string backendName = "cuda";
  std::string askedBackend;  // from the manifest, when there is one
  TaskGraph graph;
  if (args.has("run-manifest")) {
    RunManifestSpec spec;
    if (Status s = loadRunManifest(args.get("run-manifest"), spec); !s) { std::cerr << "Error: " << s.message() << "\n"; return 4; }
    if (Status s = buildTaskGraph(spec, graph); !s) { std::cerr << "Error: " << s.message() << "\n"; return 4; }
    askedBackend = spec.backendName;
  } else {
    const bool hasRoot = args.has("artifact-root"), hasKernel = args.has("kernel");
    if (hasRoot == hasKernel) { std::cerr << "Error: provide exactly one of --artifact-root or --kernel\n"; return 4; }
    KernelArtifact artifact;
    if (hasRoot) {
      if (Status s = loadArtifactFromRoot(args.get("artifact-root"), artifact); !s) { std::cerr << "Error: " << s.message() << "\n"; return 4; }
    } else {
      const std::string kind = args.get("kernel-kind", "mix");
      if (kind != "vec" && kind != "cube" && kind != "mix") { std::cerr << "Error: unsupported kernel kind: " << kind << "\n"; return 4; }
      CompileRequest request;
      request.kernelSource = args.get("kernel");
      request.kernelName = args.get("name");
      request.outputDir = args.get("output", "./build/runtime-session-artifact");
      request.socVersion = args.get("soc", "sm_100a");
      if (Status s = compileArtifact(request, artifact); !s) { std::cerr << "Error: " << s.message() << "\n"; return 4; }
    }
    std::cout << "artifact.kernel_name=" << artifact.kernelName << "\n";
    std::cout << "artifact.root=" << artifact.artifactRoot << "\n";
    std::cout << "artifact.manifest=" << artifact.manifestPath << "\n";
    std::cout << "artifact.soc=" << artifact.socVersion << "\n";
    RuntimeTask task;
    task.taskId = args.get("task-id", "main");
    task.artifact = artifact;
    if (Status s = graph.addTask(task); !s) { std::cerr << "Error: " << s.message() << "\n"; return 4; }
  }

  std::shared_ptr<ExecutionBackendDriver> driver;
  const std::string testing = args.get("testing-driver");
  if (testing.empty()) {
    const char *dev = std::getenv("AFIR_CUDA_DEVICE");
    driver = createCudaBackendDriver(dev && *dev ? std::atoi(dev) : 0);
  } else if (testing == "success" || testing == "npu-success" || testing == "cuda-success") {
    driver = std::make_shared<SuccessfulTestingDriver>();
  } else {
    std::cerr << "Error: unsupported testing driver: " << testing << "\n";
    return 4;
  }

  ExecutionSession session(backendName, driver);
  SessionPlan plan;
  if (Status s = session.plan(graph, plan); !s) { std::cerr << "Error: " << s.message() << "\n"; return 2; }
  std::cout << "session.plan.tasks=" << plan.orderedTaskIds.size() << "\n";
  for (size_t i = 0; i < plan.orderedTaskIds.size(); ++i) std::cout << "session.plan[" << i << "]=" << plan.orderedTaskIds[i] << "\n";
  if (!args.flag("run")) return 0;

  // Session directories and retained profiles live under the temp directory; each root keeps its last 20.
  constexpr size_t kSessionLimit = 20;
  const char *tmp = std::getenv("TMPDIR");
  const std::string tmpRoot = tmp && *tmp ? tmp : "/tmp";
  const std::string workRoot = tmpRoot + "/afir-cuda-runtime";
  const std::string retainRoot = tmpRoot + "/afir-cuda-runtime-profiles";
  if (Status s = prepareRetainedRootForNewSession(workRoot, kSessionLimit); !s) { std::cerr << "Error: " << s.message() << "\n"; return 4; }

  SessionRunSummary summary = session.run(graph);
  if (!summary.success) {
    printRunError(session, askedBackend, summary);
    return 2;
  }
  std::string retainedSummary;
  if (!summary.profileTrace.events.empty()) {
    RetainedProfileArtifacts kept;
    Status s = prepareRetainedRootForNewSession(retainRoot, kSessionLimit);
    if (s) s = retainProfileArtifacts(summary.profileTrace, retainRoot, kept);
    if (!s) {
      summary.success = false;
      summary.errorStage = "profiling";
      summary.errorMessage = s.message();
      printRunError(session, askedBackend, summary);
      return 2;
    }
    summary.profileTrace = kept.trace;
    summary.profileArtifactPaths.clear();
    for (const ProfileEvent &ev : kept.trace.events) summary.profileArtifactPaths.push_back(ev.artifactPath);
    retainedSummary = kept.summaryPath;
  }
  printBackend(std::cout, session, askedBackend);
  std::cout << "session.result=success\n";
  if (summary.validationRan && summary.validationPassed) std::cout << "session.validation=pass\n";
  std::cout << "session.profile.session_id=" << summary.profileTrace.sessionId << "\n";
  std::cout << "session.profile.count=" << summary.profileArtifactPaths.size() << "\n";
  for (size_t i = 0; i < summary.profileArtifactPaths.size(); ++i)
    std::cout << "session.profile[" << i << "]=" << summary.profileArtifactPaths[i] << "\n";
  if (!retainedSummary.empty()) std::cout << "session.profile.summary=" << retainedSummary << "\n";
  for (const auto &ev : summary.profileTrace.events) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "%.3f", ev.score);
    std::cout << "session.profile.score." << ev.taskId << "=" << buf << "\n";
  }
  for (const auto &kv : summary.profileTrace.attributes) std::cout << "session.runtime.attribute." << kv.first << "=" << kv.second << "\n";
  for (const auto &kv : summary.profileTrace.counters) std::cout << "session.runtime.counter." << kv.first << "=" << kv.second << "\n";
  return 0;
}
