// Loop template of elementwise groups with an operand read through a transposed view, shared by the prebuilt kernels
// (elementwise.cu) and the kernels generated per group (also compiled at run time: no host header).
#pragma once

#include "kernels/elementwise_skel.cuh"
#include "kernels/reg_block.cuh"

namespace afir {
namespace kernels {

// ---- block variant: groups with an operand read through a transposed view -----------------------------------
// When a view's unit stride runs along the second-to-last iteration dim (out[n, m] = f(a[m, n], ...)), the kernel
// above would fall back to element-wise accesses.  Here every thread owns an E x E block of the last two dims
// (E = 16 / element bytes): row-major views are read as E row pieces of 16 bytes, transposed views as E pieces
// along their own rows followed by a register transpose, views that are constant along the inner dim as one
// element per row; the body runs on the block and E 16-byte row pieces are stored.  Lanes are arranged so that a
// warp's stores and row-major loads cover whole 128-byte lines and its transposed loads 64-byte pieces.
// Ragged edge blocks are done element by element in the same kernel.
enum BlockViewKind : int { kViewRowMajor = 0, kViewTransposed = 1, kViewInnerBroadcast = 2 };

struct EbParams {
  const char *vbase[kMaxViews];
  long long s0[kMaxViews], s1[kMaxViews], s2[kMaxViews];  // element strides per iteration dim
  int kind[kMaxViews];
  int numViews;
  char *obase;
  long long os0, os1;
  long long d1, d2;
  unsigned int tilesX, tilesY;
  unsigned long long numTiles;  // batches x tilesY x tilesX
  BodyProgram prog;
};

// The loop: CTAs of 256 threads (2 x 4 warps, each 4 x 8 blocks) walk the tiles.  NVL = views actually loaded (<= B::kViews).
template <class P, class B, int NVL>
__device__ __forceinline__ void elementwiseBlocksTiles(const EbParams &prm) {
  constexpr int NV = B::kViews;
  constexpr int EB = sizeof(typename P::Scalar);
  using RB = RegBlock<EB>;
  constexpr int E = RB::kEdge;
  constexpr int kTileRows = 2 * 4 * E, kTileCols = 4 * 8 * E;  // 2 x 4 warps, each 4 x 8 blocks
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int bi = (warp >> 2) * 4 + (lane >> 3);
  const int bj = (warp & 3) * 8 + (lane & 7);
  for (unsigned long long t = blockIdx.x; t < prm.numTiles; t += gridDim.x) {
    const unsigned int tx = static_cast<unsigned int>(t % prm.tilesX);
    const unsigned long long rest = t / prm.tilesX;
    const unsigned int ty = static_cast<unsigned int>(rest % prm.tilesY);
    const long long b = static_cast<long long>(rest / prm.tilesY);
    const long long r0 = static_cast<long long>(ty) * kTileRows + static_cast<long long>(bi) * E;
    const long long c0 = static_cast<long long>(tx) * kTileCols + static_cast<long long>(bj) * E;
    if (r0 >= prm.d1 || c0 >= prm.d2) continue;
    char *orow = prm.obase + (b * prm.os0 + r0 * prm.os1 + c0) * EB;
    if (r0 + E <= prm.d1 && c0 + E <= prm.d2) {
      uint4 raw[NVL][E];
#pragma unroll
      for (int k = 0; k < NVL; ++k) {
        if (k >= prm.numViews) {
#pragma unroll
          for (int r = 0; r < E; ++r) raw[k][r] = make_uint4(0u, 0u, 0u, 0u);
          continue;
        }
        const char *base = prm.vbase[k] + b * prm.s0[k] * EB;
        if (prm.kind[k] == kViewRowMajor) {
          const char *src = base + (r0 * prm.s1[k] + c0) * EB;
#pragma unroll
          for (int r = 0; r < E; ++r) raw[k][r] = loadStream16(src + r * prm.s1[k] * EB);
        } else if (prm.kind[k] == kViewTransposed) {
          uint4 cols[E];
          const char *src = base + (c0 * prm.s2[k] + r0) * EB;
#pragma unroll
          for (int c = 0; c < E; ++c) cols[c] = loadStream16(src + c * prm.s2[k] * EB);
          RB::transpose(cols, raw[k]);
        } else {
#pragma unroll
          for (int r = 0; r < E; ++r) {
            const unsigned int s = P::splat(base + (r0 + r) * prm.s1[k] * EB).bits();
            raw[k][r] = make_uint4(s, s, s, s);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < E; ++r) {
        Vec16<P> o;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          P vals[NV];
#pragma unroll
          for (int k = 0; k < NV; ++k) {
            unsigned int bits = 0u;
            if (k < NVL) bits = q == 0 ? raw[k][r].x : q == 1 ? raw[k][r].y : q == 2 ? raw[k][r].z : raw[k][r].w;
            vals[k] = P::fromBits(bits);
          }
          o.p[q] = B::template eval<P>(vals, prm.prog);
        }
        storeStream16(orow + r * prm.os1 * EB, o.raw());
      }
    } else {
      for (int r = 0; r < E && r0 + r < prm.d1; ++r)
        for (int c = 0; c < E && c0 + c < prm.d2; ++c) {
          P vals[NV];
#pragma unroll
          for (int k = 0; k < NV; ++k) {
            vals[k] = P::fromBits(0u);
            if (k < NVL && k < prm.numViews)
              vals[k] = P::splat(prm.vbase[k] + (b * prm.s0[k] + (r0 + r) * prm.s1[k] + (c0 + c) * prm.s2[k]) * EB);
          }
          storeScalar<P>(orow + (r * prm.os1 + c) * EB, B::template eval<P>(vals, prm.prog));
        }
    }
  }
}

} // namespace kernels
} // namespace afir
