#include "execution/artifact_compiler.h"

#include <sys/stat.h>

#include <cerrno>
#include <cstring>
#include <fstream>

#include "codegen/nvrtc_compile.h"
#include "runtime/descriptor.h"
#include "support/tiling_schema.h"

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
} // namespace

Status compileArtifact(const CompileRequest &request, KernelArtifact &artifact) {
  if (request.kernelSource.empty()) return Status::error("kernel source path is required");
  if (request.outputDir.empty()) return Status::error("output directory is required");
  const bool knownArch = request.arch == "sm_100a" || request.arch.find("dav-") == 0;
  if (!knownArch) return Status::error("unsupported arch '" + request.arch + "' (this library is sm_100a only)");
  std::vector<uint8_t> src;
  if (Status s = readFileBytes(request.kernelSource, src); !s) return s;
  LaunchDescriptor desc;
  if (Status s = parseDescriptorBinary(src.data(), src.size(), desc); !s)
    return Status::error(request.kernelSource + ": " + s.message());
  const std::string name = request.kernelName.empty() ? desc.kernel : request.kernelName;
  if (desc.kernel != name)
    return Status::error(request.kernelSource + ": defines kernel '" + desc.kernel + "', not '" + name + "'");
  if (!makeDirs(request.outputDir)) return Status::error("cannot create " + request.outputDir);
  // The compile step proper: generate the group's kernel source and compile it for sm_100a (NVRTC, no GPU
  // needed), as the reference generates AscendC and runs bisheng on it
  // (lib/Runtime/Artifact/VecCubeArtifactBackend.cpp:123-189).  Matmul and bare-transpose groups are kernels of
  // the library itself and get a descriptor-only container.
  std::vector<uint8_t> bin;
  std::string codegenNote = "library";
  std::string sourcePath;
  if (src.size() >= 4 && std::memcmp(src.data(), "AFCU", 4) == 0) {
    bin = src;
    codegenNote = containerCode(src.data(), src.size()).cubinLen ? "generated" : "library";
  } else {
    const std::string srcText(src.begin(), src.end());
    const std::string embedded = embeddedDescriptorJson(srcText);
    codegen::GeneratedKernel kernel = codegen::generateKernelSource(desc);
    // A kernel source file (afir-translate -mlir-to-cann): THAT text is what gets compiled, not a regenerated one;
    // the descriptor it carries says how to launch it.  A source file of a library group holds no kernel.
    if (!embedded.empty() && kernel.supported) {
      if (srcText.find("extern \"C\" __global__") != std::string::npos) kernel.source = srcText;
      else { kernel.supported = false; kernel.whyNot = "the source file defines no kernel"; }
    }
    const std::string descriptorText = embedded.empty() ? srcText : embedded;
    std::vector<uint8_t> cubin;
    std::string source;
    if (!kernel.supported) {
      codegenNote = "library (" + kernel.whyNot + ")";
    } else {
      codegen::CompiledKernel compiled;
      if (Status s = codegen::compileToCubin(kernel, compiled); !s) {
        // a compiler that cannot be loaded is not the kernel's fault: the group then runs on the library's kernels;
        // source that does not compile is a bug and fails the step
        if (!codegen::nvrtcUnavailableReason().empty()) codegenNote = "library (" + s.message() + ")";
        else return Status::error(request.kernelSource + ": " + s.message());
      } else {
        cubin = std::move(compiled.cubin);
        source = kernel.source;
        codegenNote = "generated";
        if (!compiled.log.empty()) {  // warnings, or the register / spill report asked for with AFIR_CUDA_NVRTC_PTXAS_INFO=1
          std::ofstream log(request.outputDir + "/" + name + ".compile.log", std::ios::trunc);
          log << compiled.log << "\n";
        }
        sourcePath = request.outputDir + "/" + name + ".cu";
        std::ofstream os(sourcePath, std::ios::trunc);
        os << source;
        if (!os) return Status::error("cannot write " + sourcePath);
      }
    }
    bin = wrapDescriptorContainer(descriptorText, cubin, source);
  }
  const std::string binPath = request.outputDir + "/" + name + ".bin";
  {
    std::ofstream os(binPath, std::ios::binary | std::ios::trunc);
    os.write(reinterpret_cast<const char *>(bin.data()), static_cast<std::streamsize>(bin.size()));
    if (!os) return Status::error("cannot write " + binPath);
  }
  const std::string manifestPath = request.outputDir + "/manifest.txt";
  const bool matmul = desc.kernelClass == KernelClass::Matmul;
  {
    std::ofstream os(manifestPath, std::ios::trunc);
    os << "kernel_name=" << desc.kernel << "\n"
       << "soc_version=" << request.socVersion << "\n"
       << "kernel_kind=" << (matmul ? "mix" : "vec") << "\n"
       << "kernel_class=" << kernelClassName(desc.kernelClass) << "\n"
       << "device_binary_path=" << binPath << "\n"
       << "manifest_path=" << manifestPath << "\n"
       << "codegen=" << codegenNote << "\n";
    if (!sourcePath.empty()) os << "kernel_source_path=" << sourcePath << "\n";
    if (!os) return Status::error("cannot write " + manifestPath);
  }
  artifact = KernelArtifact();
  artifact.kernelName = desc.kernel;
  artifact.kernelKind = matmul ? KernelKind::Mix : KernelKind::Vec;
  artifact.socVersion = request.socVersion;
  artifact.artifactRoot = request.outputDir;
  artifact.deviceBinaryPath = binPath;
  artifact.manifestPath = manifestPath;
  return Status::success();
}

} // namespace afir
