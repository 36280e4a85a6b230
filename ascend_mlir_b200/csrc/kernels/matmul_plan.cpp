#include "kernels/matmul_plan.h"

#include <algorithm>

namespace afir {
namespace kernels {
namespace {

constexpr int kTileN = 256, kTileK = 64;
constexpr int kBStageBytes = kTileN * kTileK * 2;

int64_t ceilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

} // namespace

bool matmulPlannerSupports(const MatmulProblem &p) {
  return p.M > 0 && p.N > 0 && p.K > 0 && p.batchShape.empty() && p.inElemBytes == 2 && p.M < (1ll << 31) && p.N < (1ll << 31) &&
         p.K < (1ll << 31);
}

std::string buildMatmulPlan(const MatmulProblem &problem, const MatmulHints &hints, int smCount, MatmulPlan &plan) {
  if (!problem.batchShape.empty()) return "matmul planner: batched problems are not supported";
  if (problem.inElemBytes != 2) return "matmul planner: operands must be f16 or bf16";
  if (!matmulPlannerSupports(problem)) return "matmul planner: M, N and K must be positive and below 2^31";
  if (hints.variant < 0 || hints.variant > 3) return "matmul planner: variant hint must be 0 (choose), 1, 2 or 3";
  if (smCount < 1) smCount = 1;

  plan = MatmulPlan();
  // 256-row tiles halve the operand bytes moved into shared memory per flop and are the default whenever they
  // keep at least half of the SMs busy; below that, 128-row tiles put a small problem on twice as many SMs.
  // Measured on B200 (K = N = 8192, bf16): 8192^3 M-sharded over 8 GPUs (M = 1024) is 128 tiles of 256 x 256 in one
  // wave, 101 us, against 256 tiles of 128 x 256 in two waves, 112 us; the same order holds at M = 2048 (196 vs 215
  // us), 4096 (396 vs 442 us) and 8192 (764 vs 866 us).  (The earlier rule, 256-row tiles only when there is one
  // per SM, chose the slower variant at M = 1024.)
  // The tile can also be narrower than 256 columns (a hint only): 4 x 37 = 148 tiles of 256 x 224 would fill the
  // 148 SMs exactly where 4 x 32 = 128 tiles of 256 x 256 leave 20 idle, but measured a 224-column tile takes as
  // long as a 256-column one (100.3 us vs 103.1 us at M = 1024, 396 vs 385 us at M = 4096, 727 vs 767 us at
  // M = 8192): the B stage is loaded 256 columns wide either way and the kernel is not MMA-issue bound, so
  // narrowing buys nothing and is never chosen by default.
  // The CTA pair works a 256 x 256 tile in a little over half the time one SM needs (measured: 0.55 of it), and half
  // as many pairs as SMs share the tiles: it is chosen where that still comes out ahead because the tiles divide
  // better over 74 pairs than over 148 SMs.  Measured (us per launch, one CTA per SM / pairs): M = 8192, 1024 tiles,
  // 7 waves against 14 rounds: 775 / 855; M = 4096, 512 tiles, 4 waves against 7 rounds: **390 / 381**; M = 2048,
  // 256 tiles, 2 against 4: 195 / 206; M = 1024, 128 tiles, 1 against 2: 100 / 108.  It cannot take B as [N, K], whose
  // tiles it would have to split along K-major rows.
  const int64_t ctasWanted = hints.blockDim > 0 ? hints.blockDim : smCount;
  const int64_t tiles256 = ceilDiv(problem.M, 256) * ceilDiv(problem.N, kTileN);
  MatmulVariant v = 2 * tiles256 >= smCount ? MatmulVariant::Rows256 : MatmulVariant::Rows128;
  if (v == MatmulVariant::Rows256 && hints.variant == 0 && hints.blockDim <= 0 && hints.tileN <= 0 && !problem.transposeB &&
      smCount >= 2) {
    const double single = static_cast<double>(ceilDiv(tiles256, smCount));
    const double pair = 0.55 * static_cast<double>(ceilDiv(tiles256, smCount / 2));
    if (pair < 0.99 * single) v = MatmulVariant::CtaPair;
  }
  if (hints.variant != 0) v = static_cast<MatmulVariant>(hints.variant);
  if (v == MatmulVariant::CtaPair && problem.transposeB) v = MatmulVariant::Rows256;
  int tileN = kTileN;
  if (hints.tileN > 0 && v != MatmulVariant::CtaPair) {
    if (hints.tileN != 128 && hints.tileN != 160 && hints.tileN != 192 && hints.tileN != 224 && hints.tileN != 256)
      return "matmul planner: tile width hint must be 128, 160, 192, 224 or 256";
    tileN = hints.tileN;
  }
  plan.variant = v;
  plan.tileN = tileN;
  plan.tileK = kTileK;
  switch (v) {
  case MatmulVariant::Rows128:
    plan.tileM = 128; plan.stages = 4; plan.threads = 64 + 32 * 4;
    plan.operandRingBytes = static_cast<size_t>(plan.stages) * (128 * kTileK * 2 + kBStageBytes);
    plan.epilogueOverlapsMainloop = true;
    break;
  case MatmulVariant::Rows256:
    plan.tileM = 256; plan.stages = 3; plan.threads = 64 + 32 * 8;
    plan.operandRingBytes = static_cast<size_t>(plan.stages) * (256 * kTileK * 2 + kBStageBytes);
    plan.epilogueOverlapsMainloop = false;
    break;
  case MatmulVariant::CtaPair:
    plan.tileM = 256; plan.stages = 6; plan.threads = 192;
    plan.operandRingBytes = static_cast<size_t>(plan.stages) * (128 * kTileK * 2 + kBStageBytes / 2);  // per CTA of the pair
    plan.epilogueOverlapsMainloop = true;
    break;
  }
  plan.tilesM = static_cast<int>(ceilDiv(problem.M, plan.tileM));
  plan.tilesN = static_cast<int>(ceilDiv(problem.N, plan.tileN));
  plan.kBlocks = static_cast<int>(ceilDiv(problem.K, plan.tileK));
  plan.traverse = MatmulTraverse::FirstM;
  plan.band = hints.band > 0 ? hints.band : (v == MatmulVariant::CtaPair ? 8 : 16);
  const int64_t tiles = static_cast<int64_t>(plan.tilesM) * plan.tilesN;
  int64_t ctas = ctasWanted;
  if (v == MatmulVariant::CtaPair) {
    // two CTAs per tile: an even grid, at most one pair per tile
    ctas = std::min<int64_t>(ctas, 2 * tiles);
    ctas = std::max<int64_t>(2, ctas - (ctas % 2));
  } else {
    ctas = std::max<int64_t>(1, std::min<int64_t>(ctas, tiles));
  }
  plan.blockDim = static_cast<uint32_t>(ctas);
  plan.tmemColumns = 512;
  return std::string();
}

std::string describeMatmulPlan(const MatmulPlan &p) {
  const char *variant = p.variant == MatmulVariant::Rows128 ? "rows128" : p.variant == MatmulVariant::Rows256 ? "rows256" : "cta_pair";
  return "planned_block_dim=" + std::to_string(p.blockDim) + " variant=" + variant + " traverse=" +
         (p.traverse == MatmulTraverse::FirstN ? "FIRSTN" : "FIRSTM") + " band=" + std::to_string(p.band) + " tile=" +
         std::to_string(p.tileM) + "x" + std::to_string(p.tileN) + "x" + std::to_string(p.tileK) + " stages=" +
         std::to_string(p.stages) + " tiles=" + std::to_string(p.tilesM) + "x" + std::to_string(p.tilesN) + " k_blocks=" +
         std::to_string(p.kBlocks) + " ring_bytes=" + std::to_string(p.operandRingBytes) + " tmem_cols=" +
         std::to_string(p.tmemColumns) + " overlap_epilogue=" + (p.epilogueOverlapsMainloop ? "1" : "0");
}

} // namespace kernels
} // namespace afir
