// afir-translate -mlir-to-cuda: emits the launch descriptor (<kernel>.cuda.json) of a fused-group function
// and, with --tiling-space-out, its tiling_space.json.  Counterpart of the reference's
// `afir-translate -mlir-to-cann [--tiling-space-out f.json]` (tools/afir-translate/afir-translate.cpp:19-40),
// which emits AscendC C++ instead: here the code is the prebuilt sm_100a kernel library and the translation
// unit is the descriptor that selects and parameterises a kernel of it.
// `-mlir-to-cuda-kernel` goes one step further and prints the CUDA C++ source of the group's generated kernel
// (signature (in..., out..., workspace, TilingData), the text counterpart of the reference's emitted AscendC);
// `--cubin-out` also compiles it for sm_100a with NVRTC (no GPU needed).  Matmul and bare-transpose groups run on
// the hand-written kernels of the library and have no generated source: the tool says so and exits 1.
#include <fstream>
#include <iostream>
#include <iterator>

#include "codegen/nvrtc_compile.h"
#include "front/group_analysis.h"
#include "runtime/descriptor.h"

using namespace afir;
using namespace afir::front;

int main(int argc, char **argv) {
  std::string input, output, spaceOut, function, cubinOut;
  bool toCuda = false, toKernel = false, selfContained = false;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto value = [&](const std::string &name, std::string &dst) -> bool {
      const std::string dd = "--" + name, d = "-" + name;
      if (a == dd || a == d) {
        if (i + 1 >= argc) { std::cerr << "afir-translate: " << a << " needs a value\n"; std::exit(1); }
        dst = argv[++i];
        return true;
      }
      if (a.compare(0, dd.size() + 1, dd + "=") == 0) { dst = a.substr(dd.size() + 1); return true; }
      if (a.compare(0, d.size() + 1, d + "=") == 0) { dst = a.substr(d.size() + 1); return true; }
      return false;
    };
    if (a == "-mlir-to-cuda" || a == "--mlir-to-cuda") toCuda = true;
    else if (a == "-mlir-to-cuda-kernel" || a == "--mlir-to-cuda-kernel") toKernel = true;
    else if (a == "-mlir-to-cann" || a == "--mlir-to-cann") {
      // the reference's flag, for scripts written against it: the kernel source of THIS target (CUDA C++ where the
      // reference writes AscendC C++), with the launch descriptor in a leading comment block so that the file alone is
      // what afirt_compiler_compile needs
      toKernel = true;
      selfContained = true;
    } else if (value("o", output) || value("tiling-space-out", spaceOut) || value("function", function) || value("cubin-out", cubinOut)) {
    } else if (a == "--help" || a == "-h") {
      std::cout << "USAGE: afir-translate -mlir-to-cuda <input.mlir> [-o <kernel>.cuda.json] [--tiling-space-out <file>] [--function <name>]\n"
                   "       afir-translate -mlir-to-cuda-kernel <input.mlir> [-o <kernel>.cu] [--cubin-out <kernel>.cubin] [--tiling-space-out <file>]\n";
      return 0;
    } else if (a.size() > 1 && a[0] == '-') {
      std::cerr << "afir-translate: Unknown command line argument '" << a << "'\n";
      return 1;
    } else if (input.empty()) input = a;
    else { std::cerr << "afir-translate: more than one input file\n"; return 1; }
  }
  if (!toCuda && !toKernel) { std::cerr << "afir-translate: no translation requested (use -mlir-to-cuda or -mlir-to-cuda-kernel)\n"; return 1; }
  std::string text;
  if (input.empty() || input == "-") text.assign(std::istreambuf_iterator<char>(std::cin), std::istreambuf_iterator<char>());
  else {
    std::ifstream is(input);
    if (!is) { std::cerr << "afir-translate: cannot open " << input << "\n"; return 1; }
    text.assign(std::istreambuf_iterator<char>(is), std::istreambuf_iterator<char>());
  }
  Module module;
  if (Status s = parseModule(text, module); !s) { std::cerr << (input.empty() ? "<stdin>" : input) << ": error: " << s.message() << "\n"; return 1; }
  const Func *func = nullptr;
  for (const Func &f : module.funcs)
    if (function.empty() ? module.funcs.size() == 1 : f.name == function) func = &f;
  if (!func) {
    std::cerr << "afir-translate: " << (function.empty() ? "the module holds several functions; pick one with --function" : "no function named '" + function + "'") << "\n";
    return 1;
  }
  GroupAnalysis ga;
  if (Status s = analyzeFunction(module, *func, ga); !s) { std::cerr << (input.empty() ? "<stdin>" : input) << ": error: " << s.message() << "\n"; return 1; }
  std::string desc = json::dump(ga.descriptor, 2) + "\n";
  if (toKernel) {
    LaunchDescriptor parsed;
    if (Status s = parseDescriptorJson(ga.descriptor, parsed); !s) { std::cerr << "afir-translate: " << s.message() << "\n"; return 1; }
    const codegen::GeneratedKernel kernel = codegen::generateKernelSource(parsed);
    if (!kernel.supported && !selfContained) {
      std::cerr << "afir-translate: no kernel source is generated for '" << parsed.kernel << "': " << kernel.whyNot << "\n";
      return 1;
    }
    desc = kernel.source;
    if (selfContained) {
      const std::string header = embedDescriptorComment(json::dump(ga.descriptor, -1));
      desc = kernel.supported ? header + kernel.source
                              : header + "// Kernel '" + parsed.kernel + "' is a kernel of the runtime library (" + kernel.whyNot +
                                    "): this file holds its launch descriptor only.\n";
    }
    if (!cubinOut.empty() && kernel.supported) {
      codegen::CompiledKernel compiled;
      if (Status s = codegen::compileToCubin(kernel, compiled); !s) { std::cerr << "afir-translate: " << s.message() << "\n"; return 1; }
      if (!compiled.log.empty()) std::cerr << compiled.log << "\n";
      std::ofstream os(cubinOut, std::ios::binary | std::ios::trunc);
      os.write(reinterpret_cast<const char *>(compiled.cubin.data()), static_cast<std::streamsize>(compiled.cubin.size()));
      if (!os) { std::cerr << "afir-translate: cannot write " << cubinOut << "\n"; return 1; }
    }
  }
  if (output.empty() || output == "-") std::cout << desc;
  else {
    std::ofstream os(output, std::ios::trunc);
    os << desc;
    if (!os) { std::cerr << "afir-translate: cannot write " << output << "\n"; return 1; }
  }
  if (!spaceOut.empty()) {
    std::ofstream os(spaceOut, std::ios::trunc);
    os << json::dump(ga.tilingSpace, 2) << "\n";
    if (!os) { std::cerr << "afir-translate: cannot write " << spaceOut << "\n"; return 1; }
  }
  return 0;
}
