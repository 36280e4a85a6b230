#include "codegen/nvrtc_compile.h"

#include <dlfcn.h>
#include <sys/stat.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <type_traits>

namespace afir {
namespace codegen {
namespace {

// The handful of NVRTC entry points used, resolved by name (nvrtc.h's prototypes, restated with plain types).
using nvrtcProgram = void *;
struct NvrtcApi {
  void *lib = nullptr;
  std::string reason;   // why it is unusable
  std::string libPath;  // where it was loaded from
  int (*createProgram)(nvrtcProgram *, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
  int (*destroyProgram)(nvrtcProgram *) = nullptr;
  int (*compileProgram)(nvrtcProgram, int, const char *const *) = nullptr;
  int (*getCubinSize)(nvrtcProgram, size_t *) = nullptr;
  int (*getCubin)(nvrtcProgram, char *) = nullptr;
  int (*getLogSize)(nvrtcProgram, size_t *) = nullptr;
  int (*getLog)(nvrtcProgram, char *) = nullptr;
  const char *(*getErrorString)(int) = nullptr;
};

bool isDir(const std::string &p) {
  struct stat st;
  return ::stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

std::vector<std::string> cudaRoots() {
  std::vector<std::string> roots;
  for (const char *name : {"CUDA_HOME", "CUDA_PATH", "CUDA_ROOT"})
    if (const char *v = std::getenv(name))
      if (*v) roots.push_back(v);
  roots.push_back("/usr/local/cuda");
  return roots;
}

const NvrtcApi &api() {
  static NvrtcApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    std::vector<std::string> names = {"libnvrtc.so.12", "libnvrtc.so"};
    if (const char *forced = std::getenv("AFIR_CUDA_NVRTC_LIB"))
      if (*forced) names.insert(names.begin(), forced);
    for (const std::string &root : cudaRoots())
      for (const char *leaf : {"/lib64/libnvrtc.so.12", "/lib64/libnvrtc.so", "/lib/libnvrtc.so.12"}) names.push_back(root + leaf);
    for (const std::string &n : names) {
      a.lib = ::dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (a.lib) { a.libPath = n; break; }
    }
    if (!a.lib) {
      a.reason = "libnvrtc.so.12 not found (set AFIR_CUDA_NVRTC_LIB or CUDA_HOME)";
      return;
    }
    auto sym = [&](const char *name, auto &fn) {
      fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(::dlsym(a.lib, name));
      if (!fn && a.reason.empty()) a.reason = std::string("NVRTC has no symbol ") + name;
    };
    sym("nvrtcCreateProgram", a.createProgram);
    sym("nvrtcDestroyProgram", a.destroyProgram);
    sym("nvrtcCompileProgram", a.compileProgram);
    sym("nvrtcGetCUBINSize", a.getCubinSize);
    sym("nvrtcGetCUBIN", a.getCubin);
    sym("nvrtcGetProgramLogSize", a.getLogSize);
    sym("nvrtcGetProgramLog", a.getLog);
    sym("nvrtcGetErrorString", a.getErrorString);
    if (a.reason.empty()) {
      Dl_info info;
      if (::dladdr(reinterpret_cast<void *>(a.createProgram), &info) && info.dli_fname) a.libPath = info.dli_fname;
    }
  });
  return a;
}

// Directories holding cuda_fp16.h / cuda_bf16.h (only 16-bit groups include them).
std::vector<std::string> cudaIncludeDirs(const NvrtcApi &a) {
  std::vector<std::string> dirs;
  auto add = [&](const std::string &d) {
    if (isDir(d) && std::find(dirs.begin(), dirs.end(), d) == dirs.end()) dirs.push_back(d);
  };
  if (const char *forced = std::getenv("AFIR_CUDA_INCLUDE"))
    if (*forced) add(forced);
  const size_t slash = a.libPath.rfind('/');
  if (slash != std::string::npos) {
    const std::string libDir = a.libPath.substr(0, slash);
    add(libDir + "/../include");
    add(libDir + "/../../include");
  }
  for (const std::string &root : cudaRoots()) add(root + "/include");
  return dirs;
}

} // namespace

std::string nvrtcUnavailableReason() { return api().reason; }

Status compileToCubin(const GeneratedKernel &kernel, CompiledKernel &out) {
  out = CompiledKernel();
  if (!kernel.supported) return Status::error("no kernel was generated: " + kernel.whyNot);
  const NvrtcApi &a = api();
  if (!a.reason.empty()) return Status::error("NVRTC unavailable: " + a.reason);

  std::vector<const char *> headerNames, headerSources;
  for (const EmbeddedHeader &h : embeddedHeaders()) {
    headerNames.push_back(h.name);
    headerSources.push_back(h.begin);  // NUL-terminated: a zero byte follows every embedded file
  }
  nvrtcProgram prog = nullptr;
  int rc = a.createProgram(&prog, kernel.source.c_str(), (kernel.entry + ".cu").c_str(), static_cast<int>(headerNames.size()),
                           headerSources.data(), headerNames.data());
  if (rc != 0) return Status::error(std::string("nvrtcCreateProgram: ") + a.getErrorString(rc));

  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false", "-lineinfo"};
  for (const std::string &d : kernel.defines) opts.push_back("-D" + d);
  if (!kernel.defines.empty())
    for (const std::string &dir : cudaIncludeDirs(a)) opts.push_back("--include-path=" + dir);
  // AFIR_CUDA_NVRTC_PTXAS_INFO=1: registers, spills and shared memory per kernel in the compile log
  if (const char *v = std::getenv("AFIR_CUDA_NVRTC_PTXAS_INFO"))
    if (*v && std::string(v) != "0") opts.push_back("--ptxas-options=-v");
  std::vector<const char *> optPtrs;
  for (const std::string &o : opts) optPtrs.push_back(o.c_str());
  rc = a.compileProgram(prog, static_cast<int>(optPtrs.size()), optPtrs.data());
  size_t logSize = 0;
  if (a.getLogSize(prog, &logSize) == 0 && logSize > 1) {
    out.log.resize(logSize);
    a.getLog(prog, out.log.data());
    while (!out.log.empty() && (out.log.back() == '\0' || out.log.back() == '\n')) out.log.pop_back();
  }
  if (rc != 0) {
    std::string msg = std::string("NVRTC could not compile kernel '") + kernel.entry + "': " + a.getErrorString(rc);
    if (!out.log.empty()) msg += "\n" + out.log;
    a.destroyProgram(&prog);
    return Status::error(msg);
  }
  size_t size = 0;
  rc = a.getCubinSize(prog, &size);
  if (rc == 0 && size > 0) {
    out.cubin.resize(size);
    rc = a.getCubin(prog, reinterpret_cast<char *>(out.cubin.data()));
  }
  a.destroyProgram(&prog);
  if (rc != 0 || out.cubin.empty()) return Status::error(std::string("NVRTC produced no device binary: ") + a.getErrorString(rc));
  return Status::success();
}

Status compileToCubinCached(const GeneratedKernel &kernel, std::shared_ptr<const std::vector<uint8_t>> &cubin) {
  static std::mutex mu;
  static std::map<std::string, std::shared_ptr<const std::vector<uint8_t>>> cache;
  std::string key = kernel.source;
  for (const std::string &d : kernel.defines) key += "\n#" + d;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { cubin = it->second; return Status::success(); }
  }
  CompiledKernel compiled;
  if (Status s = compileToCubin(kernel, compiled); !s) return s;
  auto made = std::make_shared<const std::vector<uint8_t>>(std::move(compiled.cubin));
  std::lock_guard<std::mutex> lock(mu);
  cubin = cache.emplace(std::move(key), std::move(made)).first->second;
  return Status::success();
}

} // namespace codegen
} // namespace afir
