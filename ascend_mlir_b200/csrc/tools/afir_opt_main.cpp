// afir-opt: reads a module in the textual MLIR subset of the fused-group front end, runs the requested
// passes and prints the module.  The pass names are the reference's (tools/afir-opt/afir-opt.cpp:28-50 registers
// them on MlirOptMain) plus --convert-afir-to-cuda, the sibling of its AFIRToASCIR conversion:
//   --mark-structured-ops               gather_dim / embedding_dim on gather generics
//   --annotate-ascendc-kernel-kind      ascendc.kernel_kind = "vec" | "cube" | "mix" on the function: from the ops'
//                                       ascendc.unit attributes where a lowering stage has set them (the reference's rule,
//                                       lib/Conversion/MarkStructuredOps/AnnotateAscendCKernelKindPass.cpp:46-82: Cube and
//                                       Vector units together = "mix"), else from the fused group
//   --annotate-mix-matmul-semantics     abi_matmul_* attributes (epilogue kind, bias, layouts) on matmul functions
//   --linalg-fuse-elementwise-ops       an elementwise / broadcast / reduction chain of generics becomes ONE generic with
//                                       the fused body (what the upstream pass leaves behind)
//   --fuse-gather-elementwise           a gather with pre- and post-ops becomes one gather generic: pre-op ->
//                                       tensor.extract -> post-ops, reading the index vector and the broadcast extras
//                                       (lib/Conversion/FuseGatherElementwise/FuseGatherElementwisePass.cpp:61-303);
//                                       both record the group as afir.fused_group; groups whose views are slices of an
//                                       argument (split / concat) and matmul epilogues keep their ops
//   --convert-afir-to-cuda              afir.cuda_kernel_class / afir.cuda_launch (descriptor JSON) on the function
//   --afir-shape-inference              result types of afir.add / sub / mul / div refined from their operands (numpy-style
//                                       trailing-aligned broadcast), carried to the users, the return op and the
//                                       function's result types (lib/Dialect/AFIR/Transforms/AFIRInferShapes.cpp:94-176)
// Structural passes of upstream MLIR that do not change what the group computes (--canonicalize, --cse,
// --afir-canonicalize, --linalg-fold-unit-extent-dims, --linalg-generalize-named-ops: the named ops of the subset,
// linalg.matmul and linalg.fill, are analysed as they are) verify and pass the module through.
//
// The reference's device-lowering stages are accepted under their own names, so that its example scripts and its
// torch pipeline (examples/*/run.sh, python/torch/framework/pipeline.py:_run_mlir_pipeline) drive this tool with
// only the tool path changed:
//   --transform-interpreter             reads the transform.named_sequence beside the function: the number of index
//                                       arguments it adds (transform.func.add_index_args = the tile parameters) and
//                                       its tile sizes / annotations are recorded on the function (afir.tile_index_args,
//                                       afir.tile_sizes, afir.schedule_annotations); no loops are materialised -- the
//                                       sm_100a kernel is generated from the fused group as a whole and its launch
//                                       parameters are tuned through the tiling space, not through scf.for nests
//   --transform-preload-library=transform-library-paths=<file>[,...]
//                                       the schedule lives in a file of its own: its named sequences are read as if they
//                                       stood beside the payload
//   --one-shot-bufferize[=opts], --ascendc-buffer-placement, --ascendc-fold-concat-alloc, --linalg-to-ascendc,
//   --ascendc-parallelize, --ascendc-prepare-for-emit
//                                       bufferisation, on-chip buffer placement, AscendC op selection, multi-core
//                                       dispatch and emit preparation have no counterpart on this target (global
//                                       memory is addressed directly, the grid is the dispatch): each verifies that
//                                       every function is still one fused group and records itself in afir.stages
//   --canonicalize-cann-signature       removes the transform sequence and records cann.num_inputs / cann.num_outputs
//                                       (the kernel-argument order inputs..., outputs..., workspace, tiling of
//                                       lib/Conversion/CanonicalizeCannSignature/CanonicalizeCannSignaturePass.cpp:57-140
//                                       is what the generated kernel takes)
// Any other flag, and any op outside the subset, is an error.
#include <fstream>
#include <iostream>
#include <iterator>
#include <set>

#include "front/fused_generic.h"
#include "front/group_analysis.h"
#include "front/shape_inference.h"

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
  const std::set<std::string> passThrough = {"canonicalize", "cse", "afir-canonicalize", "linalg-fold-unit-extent-dims",
                                             "linalg-generalize-named-ops", "allow-unregistered-dialect", "transform-preload-library"};
  const std::set<std::string> typePasses = {"afir-shape-inference"};
  // the reference's lowering stages (see the header comment)
  const std::set<std::string> loweringStages = {"one-shot-bufferize", "ascendc-buffer-placement", "ascendc-fold-concat-alloc",
                                                "linalg-to-ascendc", "ascendc-parallelize", "ascendc-prepare-for-emit"};
  const std::set<std::string> scheduleStages = {"transform-interpreter", "canonicalize-cann-signature"};
  std::vector<std::string> passes;
  std::vector<std::string> scheduleLibraries;  // --transform-preload-library=transform-library-paths=a.mlir[,b.mlir]
  std::string input, output;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "-o" || a == "--o") {
      if (i + 1 >= argc) { std::cerr << "afir-opt: -o needs a file name\n"; return 1; }
      output = argv[++i];
    } else if (a == "--help" || a == "-h") {
      std::cout << "USAGE: afir-opt [passes] <input.mlir> [-o <output.mlir>]\n";
      for (const auto &p : analysisPasses) std::cout << "  --" << p << "\n";
      for (const auto &p : scheduleStages) std::cout << "  --" << p << "\n";
      for (const auto &p : loweringStages) std::cout << "  --" << p << "\n";
      for (const auto &p : typePasses) std::cout << "  --" << p << "\n";
      for (const auto &p : passThrough) std::cout << "  --" << p << "\n";
      return 0;
    } else if (a.size() > 1 && a[0] == '-' && a != "-") {
      std::string name = a.substr(a[1] == '-' ? 2 : 1);
      const size_t eq = name.find('=');  // --one-shot-bufferize=bufferize-function-boundaries=true ...: options are not needed here
      const std::string options = eq != std::string::npos ? name.substr(eq + 1) : std::string();
      if (eq != std::string::npos) name = name.substr(0, eq);
      if (name == "transform-preload-library") {
        const std::string key = "transform-library-paths=";
        const size_t at = options.find(key);
        if (at == std::string::npos) { std::cerr << "afir-opt: --transform-preload-library needs transform-library-paths=<file>[,<file>]\n"; return 1; }
        std::string list = options.substr(at + key.size());
        const size_t stop = list.find(' ');
        if (stop != std::string::npos) list = list.substr(0, stop);
        for (size_t b = 0; b <= list.size();) {
          const size_t c = list.find(',', b);
          const std::string one = list.substr(b, c == std::string::npos ? std::string::npos : c - b);
          if (!one.empty()) scheduleLibraries.push_back(one);
          if (c == std::string::npos) break;
          b = c + 1;
        }
      }
      if (!analysisPasses.count(name) && !passThrough.count(name) && !loweringStages.count(name) && !scheduleStages.count(name) &&
          !typePasses.count(name)) {
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

  // Schedules kept in files of their own (the reference's gather example preloads step2_transform.mlir as a transform
  // library and runs the interpreter on the payload file): their named sequences join the module's; nothing of a
  // library is printed.
  for (const std::string &lib : scheduleLibraries) {
    std::ifstream is(lib);
    if (!is) { std::cerr << "afir-opt: cannot open transform library " << lib << "\n"; return 1; }
    const std::string libText((std::istreambuf_iterator<char>(is)), std::istreambuf_iterator<char>());
    Module library;
    if (Status s = parseModule(libText, library); !s) { std::cerr << lib << ": error: " << s.message() << "\n"; return 1; }
    if (library.schedules.empty()) { std::cerr << lib << ": error: the transform library holds no transform.named_sequence\n"; return 1; }
    for (TransformSchedule sched : library.schedules) {
      sched.srcBegin = sched.srcEnd = 0;  // not part of this module's text
      module.schedules.push_back(sched);
    }
  }

  // types first: the analyses below then see the refined shapes
  for (const auto &p : passes)
    if (p == "afir-shape-inference") { inferAfirShapes(module); break; }

  bool needAnalysis = false;
  for (const auto &p : passes) needAnalysis = needAnalysis || analysisPasses.count(p) || loweringStages.count(p) || scheduleStages.count(p);
  for (const auto &p : passes)
    if (p == "transform-interpreter" && module.schedules.empty()) {
      std::cerr << (input.empty() ? "<stdin>" : input) << ": error: --transform-interpreter: the module holds no transform.named_sequence\n";
      return 1;
    }
  // Functions whose ops carry ascendc.unit attributes (the buffer-level form a lowering stage leaves behind) get their
  // kernel kind from those; such a function is not a fused group on tensors and the group analysis is not asked.
  std::set<std::string> kindFromUnits;
  for (const auto &p : passes) {
    if (p != "annotate-ascendc-kernel-kind") continue;
    for (Func &f : module.funcs) {
      bool cube = false, vector = false, any = false;
      std::string bad;
      std::vector<const Op *> work;
      for (const Op &o : f.ops) work.push_back(&o);
      while (!work.empty()) {
        const Op *o = work.back();
        work.pop_back();
        for (const Op &inner : o->body) work.push_back(&inner);
        if (o->unit.empty()) continue;
        any = true;
        if (o->unit == "AiCore.Cube") cube = true;
        else if (o->unit == "AiCore.Vector") vector = true;
        else if (bad.empty()) bad = "line " + std::to_string(o->line) + ": unsupported ascendc.unit value for kernel kind: " + o->unit;
      }
      if (!bad.empty()) { std::cerr << (input.empty() ? "<stdin>" : input) << ": error: " << bad << "\n"; return 1; }
      if (!any || kindFromUnits.count(f.name)) continue;
      f.addedAttrs.push_back({"ascendc.kernel_kind", cube && vector ? "\"mix\"" : cube ? "\"cube\"" : "\"vec\""});
      kindFromUnits.insert(f.name);
    }
  }
  bool onlyKind = true;  // no other analysis pass asked for
  for (const auto &p : passes) onlyKind = onlyKind && !((analysisPasses.count(p) && p != "annotate-ascendc-kernel-kind") || loweringStages.count(p) || scheduleStages.count(p));

  std::set<std::string> rewritten;
  if (needAnalysis) {
    for (Func &f : module.funcs) {
      if (onlyKind && kindFromUnits.count(f.name)) continue;
      GroupAnalysis ga;
      if (Status s = analyzeFunction(module, f, ga); !s) { std::cerr << (input.empty() ? "<stdin>" : input) << ": error: " << s.message() << "\n"; return 1; }
      for (const auto &p : passes) {
        if (p == "mark-structured-ops") {
          for (const auto &oa : ga.opAttrs)
            for (const auto &kv : oa.second) f.ops[oa.first].addedAttrs.push_back(kv);
        } else if (p == "annotate-ascendc-kernel-kind") {
          if (!kindFromUnits.count(f.name)) f.addedAttrs.push_back(ga.funcAttrs.front());
        } else if (p == "annotate-mix-matmul-semantics") {
          for (size_t i = 1; i < ga.funcAttrs.size(); ++i) f.addedAttrs.push_back(ga.funcAttrs[i]);
        } else if (p == "linalg-fuse-elementwise-ops" || p == "fuse-gather-elementwise") {
          // The group's generics become ONE generic with the fused body (elementwise / reduction chains under the
          // first flag, a gather with its pre- and post-ops under the second).  Groups the rewrite does not cover
          // (slices of an argument, a matmul and its epilogue) keep their ops; either way the function records
          // which group it fuses into.
          const bool gatherGroup = ga.kernelClass == "gather";
          if ((p == "fuse-gather-elementwise") == gatherGroup && !rewritten.count(f.name)) {
            std::string why;
            if (fuseGenericsInPlace(module, f, ga, why)) rewritten.insert(f.name);
          }
          bool have = false;
          for (const auto &kv : f.addedAttrs) have = have || kv.first == "afir.fused_group";
          if (!have) f.addedAttrs.push_back({"afir.fused_group", "\"" + ga.kernelClass + "\""});
        } else if (p == "transform-interpreter") {
          int indexArgs = 0;
          std::string sizes, notes;
          for (const TransformSchedule &sched : module.schedules) {
            indexArgs += sched.indexArgs;
            for (const std::string &t : sched.tileSizes) sizes += (sizes.empty() ? "" : ", ") + t;
            for (const std::string &n : sched.annotations)
              if (notes.find("\"" + n + "\"") == std::string::npos) notes += (notes.empty() ? "\"" : ", \"") + n + "\"";
          }
          f.addedAttrs.push_back({"afir.tile_index_args", std::to_string(indexArgs) + " : i64"});
          f.addedAttrs.push_back({"afir.tile_sizes", escapeForAttr("[" + sizes + "]")});
          f.addedAttrs.push_back({"afir.schedule_annotations", "[" + notes + "]"});
        } else if (loweringStages.count(p)) {
          // one attribute per stage: the printer never rewrites an attribute an earlier run left on the function
          std::string key = "afir.stage.";
          for (char c : p) key.push_back(c == '-' ? '_' : c);
          f.addedAttrs.push_back({key, "true"});
        } else if (p == "canonicalize-cann-signature") {
          f.addedAttrs.push_back({"cann.num_inputs", std::to_string(ga.descriptor.getInt("num_inputs", 0)) + " : i64"});
          f.addedAttrs.push_back({"cann.num_outputs", std::to_string(ga.descriptor.getInt("num_outputs", 0)) + " : i64"});
        } else if (p == "convert-afir-to-cuda") {
          f.addedAttrs.push_back({"afir.cuda_kernel_class", "\"" + ga.kernelClass + "\""});
          f.addedAttrs.push_back({"afir.cuda_launch", escapeForAttr(json::dump(ga.descriptor))});
        }
      }
    }
  }
  for (const auto &p : passes)
    if (p == "canonicalize-cann-signature") {
      // the schedule has done its job: drop it, and the module attribute that announced it
      for (const TransformSchedule &sched : module.schedules) module.erasures.push_back({sched.srcBegin, sched.srcEnd});
      if (module.moduleAttrEnd > module.moduleAttrBegin &&
          module.source.substr(module.moduleAttrBegin, module.moduleAttrEnd - module.moduleAttrBegin).find("transform.with_named_sequence") != std::string::npos)
        module.erasures.push_back({module.moduleAttrBegin, module.moduleAttrEnd});
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
