// afir-opt: reads a module in the textual MLIR subset of the fused-group front end, runs the requested
// passes and prints the module.  The pass names are the reference's (tools/afir-opt/afir-opt.cpp:28-50 registers
// them on MlirOptMain) plus --convert-afir-to-cuda, the sibling of its AFIRToASCIR conversion:
//   --mark-structured-ops               gather_dim / embedding_dim on gather generics
//   --annotate-ascendc-kernel-kind      ascendc.kernel_kind = "vec" | "cube" | "mix" on the function
//   --annotate-mix-matmul-semantics     abi_matmul_* attributes (epilogue kind, bias, layouts) on matmul functions
//   --linalg-fuse-elementwise-ops, --fuse-gather-elementwise
//                                       fusion is carried out symbolically by the conversion; these check that the
//                                       function fuses into one group and record its size as afir.fused_group
//   --convert-afir-to-cuda              afir.cuda_kernel_class / afir.cuda_launch (descriptor JSON) on the function
// Structural passes of upstream MLIR that do not change what the group computes (--canonicalize, --cse,
// --afir-canonicalize, --afir-shape-inference, --linalg-fold-unit-extent-dims) verify and pass the module through.
// Any other flag, and any op outside the subset, is an error.
#include <fstream>
#include <iostream>
#include <iterator>
#include <set>

#include "front/group_analysis.h"

using namespace afir;
using namespace afir::front;

namespace {
std::string escapeForAttr(const std::string &s) {
  std::string out = "\"";
  for (char c : s) {
    if (c == '"' || c == '\\') out.push_back('\\');
    out.push_back(c);
  }
  return out + "\"";
}
} // namespace

int main(int argc, char **argv) {
  const std::set<std::string> analysisPasses = {"mark-structured-ops", "annotate-ascendc-kernel-kind", "annotate-mix-matmul-semantics",
                                                "linalg-fuse-elementwise-ops", "fuse-gather-elementwise", "convert-afir-to-cuda"};
  const std::set<std::string> passThrough = {"canonicalize", "cse", "afir-canonicalize", "afir-shape-inference",
                                             "linalg-fold-unit-extent-dims", "allow-unregistered-dialect"};
  std::vector<std::string> passes;
  std::string input, output;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "-o" || a == "--o") {
      if (i + 1 >= argc) { std::cerr << "afir-opt: -o needs a file name\n"; return 1; }
      output = argv[++i];
    } else if (a == "--help" || a == "-h") {
      std::cout << "USAGE: afir-opt [passes] <input.mlir> [-o <output.mlir>]\n";
      for (const auto &p : analysisPasses) std::cout << "  --" << p << "\n";
      for (const auto &p : passThrough) std::cout << "  --" << p << "\n";
      return 0;
    } else if (a.size() > 1 && a[0] == '-' && a != "-") {
      const std::string name = a.substr(a[1] == '-' ? 2 : 1);
      if (!analysisPasses.count(name) && !passThrough.count(name)) {
        std::cerr << "afir-opt: Unknown command line argument '" << a << "'\n";
        return 1;
      }
      passes.push_back(name);
    } else if (input.empty()) {
      input = a;
    } else {
      std::cerr << "afir-opt: more than one input file\n";
      return 1;
    }
  }
  std::string text;
  if (input.empty() || input == "-") text.assign(std::istreambuf_iterator<char>(std::cin), std::istreambuf_iterator<char>());
  else {
    std::ifstream is(input);
    if (!is) { std::cerr << "afir-opt: cannot open " << input << "\n"; return 1; }
    text.assign(std::istreambuf_iterator<char>(is), std::istreambuf_iterator<char>());
  }
  Module module;
  if (Status s = parseModule(text, module); !s) { std::cerr << (input.empty() ? "<stdin>" : input) << ": error: " << s.message() << "\n"; return 1; }

  bool needAnalysis = false;
  for (const auto &p : passes) needAnalysis = needAnalysis || analysisPasses.count(p);
  if (needAnalysis) {
    for (Func &f : module.funcs) {
      GroupAnalysis ga;
      if (Status s = analyzeFunction(module, f, ga); !s) { std::cerr << (input.empty() ? "<stdin>" : input) << ": error: " << s.message() << "\n"; return 1; }
      for (const auto &p : passes) {
        if (p == "mark-structured-ops") {
          for (const auto &oa : ga.opAttrs)
            for (const auto &kv : oa.second) f.ops[oa.first].addedAttrs.push_back(kv);
        } else if (p == "annotate-ascendc-kernel-kind") {
          f.addedAttrs.push_back(ga.funcAttrs.front());
        } else if (p == "annotate-mix-matmul-semantics") {
          for (size_t i = 1; i < ga.funcAttrs.size(); ++i) f.addedAttrs.push_back(ga.funcAttrs[i]);
        } else if (p == "linalg-fuse-elementwise-ops" || p == "fuse-gather-elementwise") {
          bool have = false;
          for (const auto &kv : f.addedAttrs) have = have || kv.first == "afir.fused_group";
          if (!have) f.addedAttrs.push_back({"afir.fused_group", "\"" + ga.kernelClass + "\""});
        } else if (p == "convert-afir-to-cuda") {
          f.addedAttrs.push_back({"afir.cuda_kernel_class", "\"" + ga.kernelClass + "\""});
          f.addedAttrs.push_back({"afir.cuda_launch", escapeForAttr(json::dump(ga.descriptor))});
        }
      }
    }
  }
  const std::string printed = printModule(module);
  if (output.empty() || output == "-") std::cout << printed;
  else {
    std::ofstream os(output, std::ios::trunc);
    os << printed;
    if (!os) { std::cerr << "afir-opt: cannot write " << output << "\n"; return 1; }
  }
  return 0;
}
