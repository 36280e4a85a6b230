// Host-side plan of one tcgen05 matmul launch: which kernel variant, its tile, ring depth, grid and tile order.
// The reference plans its Cube matmul the same way before it materialises tiling data
// (include/Runtime/Mix/NativeMatmulPlanner.h:9-30, lib/Runtime/Mix/NativeMatmulPlanner.cpp:56-118: supports /
// buildPlan / describePlan, hints that override the defaults, batches refused); here the choices are the B200
// kernel's: 128- or 256-row CTA tiles, or a 256-row tile over a CTA pair, one persistent CTA per SM.
// launchMatmul() launches exactly what buildMatmulPlan() returns; nothing here needs a GPU.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace afir {
namespace kernels {

enum class MatmulVariant : int {
  Rows128 = 1,   // 128 x 256 CTA tile, 4 stages, the two accumulators double-buffered (epilogue overlaps the next tile)
  Rows256 = 2,   // 256 x 256 CTA tile, 3 stages, both accumulators in use by one tile
  CtaPair = 3,   // 256 x 256 tile over two SMs (tcgen05 cta_group::2), 6 stages; opt-in
};
enum class MatmulTraverse : int { FirstM = 0, FirstN = 1 };

struct MatmulProblem {
  int64_t M = 0, N = 0, K = 0;
  std::vector<int64_t> batchShape;  // must be empty: batched matmuls are not planned (as in the reference)
  int inElemBytes = 2;              // f16 / bf16 operands
  bool transposeB = false;          // B given as [N, K]
};

struct MatmulHints {
  int variant = 0;    // 0 = choose; else a MatmulVariant value (the descriptor's launch.stages field)
  int blockDim = 0;   // 0 = one CTA per SM (capped by the number of tiles)
  int band = 0;       // 0 = default tile-rows per raster band
  int tileN = 0;      // 0 = choose; else the tile width to use (128, 160, 192, 224 or 256; single-CTA variants)
};

struct MatmulPlan {
  MatmulVariant variant = MatmulVariant::Rows128;
  MatmulTraverse traverse = MatmulTraverse::FirstM;  // tile order inside a band of `band` tile-rows
  int tileM = 128, tileN = 256, tileK = 64;           // per CTA (per CTA pair for CtaPair); tileN may be narrower than
                                                      // 256 when that fills the last wave of persistent CTAs
  int stages = 4;
  int threads = 192;
  int tilesM = 0, tilesN = 0, kBlocks = 0;
  int band = 16;
  uint32_t blockDim = 1;   // persistent CTAs launched
  size_t operandRingBytes = 0;  // shared memory held by the operand stages of one CTA
  int tmemColumns = 512;
  bool epilogueOverlapsMainloop = false;  // a free accumulator exists while the next tile is multiplied
};

bool matmulPlannerSupports(const MatmulProblem &problem);
// Returns an empty string and fills `plan`, or the reason the problem is refused.
std::string buildMatmulPlan(const MatmulProblem &problem, const MatmulHints &hints, int smCount, MatmulPlan &plan);
// One line, stable across runs (the launch trace prints it).
std::string describeMatmulPlan(const MatmulPlan &plan);

} // namespace kernels
} // namespace afir
