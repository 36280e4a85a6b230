// Compiling a kernel for this runtime: validate the launch descriptor, generate the CUDA source of the fused
// group's kernel (codegen/kernel_source), compile it for sm_100a with NVRTC (codegen/nvrtc_compile), seal
// descriptor + device binary + source in the .bin container and write the artifact manifest (the keys the
// reference writes in lib/Runtime/Artifact/VecCubeArtifactBackend.cpp:98-102, plus `codegen` and
// `kernel_source_path`).  Counterpart of the reference's ArtifactCompiler::compile
// (lib/Runtime/Artifact/ArtifactCompiler.cpp:22-63), which shells out to bisheng.  Matmul and bare-transpose
// groups are kernels of the library itself (hand-written tcgen05 / register-block code): their container holds
// the descriptor only.
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
