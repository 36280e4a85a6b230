// Run manifest (JSON) and artifact root (out/manifest.txt key=value) loaders.  Field names as in the
// reference (lib/Runtime/Artifact/RunManifest.cpp:92-290; artifact keys
// lib/Runtime/Artifact/VecCubeArtifactBackend.cpp:98-102): backend, artifact_root, task_id, dependencies,
// inputs/outputs/expected_outputs[{name, path | source:"task_output", upstream_task, upstream_output, shape,
// dtype}], tiling{schema, params, binary}, block_dim, workspace_size, profiling, atol, rtol, tasks[].
// Backend "cuda" runs on the GPU; "sim" and "npu" (the reference's names) are accepted and run there too.
#pragma once

#include <string>

#include "execution/task_graph.h"

namespace afir {

struct RunManifestSpec {
  std::string backendName = "cuda";
  std::vector<RuntimeTask> tasks;
};

Status loadArtifactFromRoot(const std::string &root, KernelArtifact &out);
Status loadRunManifest(const std::string &path, RunManifestSpec &out);
Status buildTaskGraph(const RunManifestSpec &spec, TaskGraph &graph);

} // namespace afir
