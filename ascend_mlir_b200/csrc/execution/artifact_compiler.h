// "Compiling" a kernel for this runtime: validate the launch descriptor against the prebuilt sm_100a
// kernel library, seal it in the .bin container and write the artifact manifest (the keys the reference
// writes in lib/Runtime/Artifact/VecCubeArtifactBackend.cpp:98-102).  Counterpart of the reference's
// ArtifactCompiler::compile (lib/Runtime/Artifact/ArtifactCompiler.cpp:22-63), which shells out to bisheng.
#pragma once

#include <string>

#include "execution/task_graph.h"

namespace afir {

struct CompileRequest {
  std::string kernelSource;  // launch descriptor (.cuda.json) or an existing container
  std::string outputDir;
  std::string kernelName;    // empty: take the descriptor's
  std::string socVersion = "sm_100a";
  std::string arch = "sm_100a";
};

Status compileArtifact(const CompileRequest &request, KernelArtifact &artifact);

} // namespace afir
