// Kernel generator: turns the launch descriptor of one fused group into the CUDA C++ source of its device
// kernel.  This is the translate step of the reference (lib/Target/CannKernel/CannTranslation.cpp:2487-2694 emits
// AscendC C++ per fused group; the TilingData struct at :1957-1985, the kernel signature at :2045-2123): here the
// emitted text is a sm_100a kernel with the same argument convention,
//
//     extern "C" __global__ void <kernel>(in..., out..., workspace, TilingData t)
//
// (lib/Conversion/CanonicalizeCannSignature/CanonicalizeCannSignaturePass.cpp:57-140), whose TilingData is the
// descriptor's all-int64 field list (tile parameters first, then dim_arg<N>_<D>,
// lib/Conversion/AscendCPrepareForEmit/AscendCPrepareForEmitPass.cpp:200-216) followed by eight words the
// runtime fills in at launch: a row window of the leading iteration dim and six launch-plan values.
//
// The fused body becomes straight-line code (one call per arith op, rounding after each); index arithmetic is
// resolved symbolically from the views (shapes, maps, slice offsets): iteration dims that every view walks
// contiguously are merged at generation time and literal extents fold into constants, dynamic ones are read
// from TilingData.  The loops themselves are the function templates of kernels/*_skel.cuh, the same ones the
// prebuilt kernels instantiate.  No CUDA is needed to generate source; compiling it is codegen/nvrtc_compile.
#pragma once

#include <string>
#include <vector>

#include "runtime/descriptor.h"

namespace afir {
namespace codegen {

// Words appended to the descriptor's tiling fields in the generated TilingData.
constexpr int kHiddenTilingWords = 8;
enum HiddenWord : int { kRowBegin = 0, kRowEnd = 1, kPlan0 = 2 };  // kPlan0 .. kPlan0 + 5: launch-plan values

// What the plan words mean per kernel class (the launcher fills them, the generated kernel reads them).
//   elementwise: none.
//   row_reduce, entry <kernel>:           p0 = 16-byte access (0/1), p1 = column slices, p2 = vectors per slice,
//                                         p3 = lanes per row
//   row_reduce, entry <kernel>__staged:   p0 = ring stages per warp, p1 = bytes per stage
//   row_reduce, entry <kernel>__finalize: p1 = column slices
//   gather (rows): p0 = vectors in flight per thread (1 or 2); p1, p2 = multiply-shift constants (magic | shift << 32)
//                  of the division by the row length in 16-byte vectors (p1) and in elements (p2); entry
//                  <kernel>__one is the same kernel without the two-in-flight path (fewer registers), launched
//                  when p0 = 1

struct GeneratedKernel {
  bool supported = false;
  std::string whyNot;              // when !supported: what in the group the generator does not cover
  std::string source;              // one translation unit
  std::string entry;               // the main kernel: the descriptor's kernel name
  bool hasStaged = false;          // row_reduce: <entry>__staged exists (exactly one streamed view)
  bool hasFinalize = false;        // row_reduce: <entry>__finalize exists
  bool hasSingleVectorEntry = false;  // gather: <entry>__one exists (the plan with one vector per thread in flight)
  bool hasTransposedOperand = false;  // elementwise: a group reads an operand through a transposed view (register-block loop)
  std::vector<std::string> defines;  // AFIR_CG_F16 / AFIR_CG_BF16 as the group's element type needs
};

GeneratedKernel generateKernelSource(const LaunchDescriptor &d);

// An empty kernel of this name is in every generated module whose kernels start with gridDependencyPrologue()
// (kernels/ew_common.cuh); the runtime launches only such modules with programmatic stream serialisation, so a
// device binary from before that convention keeps the ordinary launch.
constexpr const char *kGridDependencyMarker = "afir_waits_for_grid_dependencies";

// An empty kernel of this name is in every generated elementwise module whose kernel holds the register-block loop of
// groups with a transposed operand: that kernel is compiled for CTAs of at most 256 threads, so the runtime launches it
// with exactly 256 whatever the tiling says.
constexpr const char *kRegisterBlockMarker = "afir_ctas_of_256_threads";

} // namespace codegen
} // namespace afir
