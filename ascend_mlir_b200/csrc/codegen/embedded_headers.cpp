// The device headers a generated kernel includes, embedded byte for byte from the source tree at build time
// (.incbin resolves against the compiler's -I directories), so that what NVRTC compiles at run time is exactly
// what nvcc compiled into the prebuilt kernels.
#include "codegen/nvrtc_compile.h"

#define AFIR_EMBED(symbol, path)                                                                         \
  __asm__(".section .rodata\n"                                                                           \
          ".global " #symbol "_begin\n" #symbol "_begin:\n"                                              \
          ".incbin \"" path "\"\n"                                                                       \
          ".global " #symbol "_end\n" #symbol "_end:\n"                                                  \
          ".byte 0\n"                                                                                    \
          ".previous\n");                                                                                \
  extern "C" const char symbol##_begin[];                                                                \
  extern "C" const char symbol##_end[];

AFIR_EMBED(afir_hdr_kernels, "kernels/kernels.h")
AFIR_EMBED(afir_hdr_grid_dependency, "kernels/grid_dependency.cuh")
AFIR_EMBED(afir_hdr_ew_common, "kernels/ew_common.cuh")
AFIR_EMBED(afir_hdr_elementwise_skel, "kernels/elementwise_skel.cuh")
AFIR_EMBED(afir_hdr_elementwise_blocks_skel, "kernels/elementwise_blocks_skel.cuh")
AFIR_EMBED(afir_hdr_reg_block, "kernels/reg_block.cuh")
AFIR_EMBED(afir_hdr_row_reduce_skel, "kernels/row_reduce_skel.cuh")
AFIR_EMBED(afir_hdr_gather_skel, "kernels/gather_skel.cuh")

namespace afir {
namespace codegen {

const std::vector<EmbeddedHeader> &embeddedHeaders() {
  static const std::vector<EmbeddedHeader> headers = {
      {"kernels/kernels.h", afir_hdr_kernels_begin, afir_hdr_kernels_end},
      {"kernels/grid_dependency.cuh", afir_hdr_grid_dependency_begin, afir_hdr_grid_dependency_end},
      {"kernels/ew_common.cuh", afir_hdr_ew_common_begin, afir_hdr_ew_common_end},
      {"kernels/elementwise_skel.cuh", afir_hdr_elementwise_skel_begin, afir_hdr_elementwise_skel_end},
      {"kernels/elementwise_blocks_skel.cuh", afir_hdr_elementwise_blocks_skel_begin, afir_hdr_elementwise_blocks_skel_end},
      {"kernels/reg_block.cuh", afir_hdr_reg_block_begin, afir_hdr_reg_block_end},
      {"kernels/row_reduce_skel.cuh", afir_hdr_row_reduce_skel_begin, afir_hdr_row_reduce_skel_end},
      {"kernels/gather_skel.cuh", afir_hdr_gather_skel_begin, afir_hdr_gather_skel_end},
  };
  return headers;
}

} // namespace codegen
} // namespace afir
