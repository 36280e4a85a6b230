// Compiles a generated kernel to a sm_100a device binary with NVRTC, the compile step of the reference
// (lib/Runtime/Artifact/VecCubeArtifactBackend.cpp:123-189 shells out to bisheng for the AscendC source; here the
// compiler is a library call and needs no GPU).  NVRTC is loaded with dlopen on first use, so the runtime library
// itself has no link-time dependency on it; the headers a generated kernel includes (kernels/kernels.h and the
// *_skel.cuh loop templates) are embedded in this library and handed to NVRTC from memory.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "codegen/kernel_source.h"
#include "common/status.h"

namespace afir {
namespace codegen {

struct CompiledKernel {
  std::vector<uint8_t> cubin;
  std::string log;  // compiler messages (warnings), possibly empty
};

// Why NVRTC cannot be used in this process ("" when it can): library not found, or a symbol missing.
std::string nvrtcUnavailableReason();

Status compileToCubin(const GeneratedKernel &kernel, CompiledKernel &out);

// compileToCubin behind a process-wide cache keyed by the source text: executors that meet the same group
// (several executors in one process, the same descriptor run again) compile it once.
Status compileToCubinCached(const GeneratedKernel &kernel, std::shared_ptr<const std::vector<uint8_t>> &cubin);

// The embedded headers, by include name (for tools that print or save what a generated kernel is compiled against).
struct EmbeddedHeader { const char *name; const char *begin; const char *end; };
const std::vector<EmbeddedHeader> &embeddedHeaders();

} // namespace codegen
} // namespace afir
