// 2-D transpose out[c, r] = in[r, c] (permutation generics,
// lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:1275-1290).  HBM-bound.
//
// Main kernel (16-byte-aligned operands): every thread owns an E x E block of elements, E = 16 / element
// bytes (8 x 8 for 16-bit, 4 x 4 for 32-bit types).  It reads the block as E row pieces of 16 bytes, all E
// loads in flight at once, transposes it in registers (byte permutes for 16-bit elements, pure renaming for
// 32-bit ones) and writes E row pieces of 16 bytes of the output.  Lane l of a warp takes block row l % 8 and
// block column l / 8, so one store instruction of a warp writes four full 128-byte lines and one load
// instruction reads eight 64-byte pieces; no shared memory is involved, so the kernel never competes for
// shared-memory bandwidth and holds 128 bytes per thread in flight.  The eight warps of a CTA form a
// WR x WC grid of warp tiles (a launch parameter); edge blocks that are not whole fall back to guarded
// element accesses inside the same kernel.
//
// Fallback kernel (unaligned bases or row strides): a 64 x 64 tile goes through padded shared memory with
// element-wise accesses that are coalesced on both sides.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <type_traits>

#include "kernels/ew_common.cuh"
#include "kernels/kernels.h"
#include "kernels/launch_util.h"
#include "kernels/reg_block.cuh"

namespace afir {
namespace kernels {
namespace {

constexpr int kTile = 64;

template <typename T>
__global__ void __launch_bounds__(256) transposeKernel(const T *__restrict__ in, T *__restrict__ out, long long rows,
                                                       long long cols, long long inStride, long long outStride,
                                                       unsigned int tilesX, unsigned long long numTiles) {
  gridDependencyPrologue();
  __shared__ T tile[kTile][kTile + 1];
  const int tx = threadIdx.x & 63;  // fast index inside the tile
  const int ty = threadIdx.x >> 6;  // 0..3
  for (unsigned long long t = blockIdx.x; t < numTiles; t += gridDim.x) {
    const long long r0 = static_cast<long long>(t / tilesX) * kTile;
    const long long c0 = static_cast<long long>(t % tilesX) * kTile;
#pragma unroll 4
    for (int y = ty; y < kTile; y += 4) {
      const long long r = r0 + y, c = c0 + tx;
      if (r < rows && c < cols) tile[y][tx] = in[r * inStride + c];
    }
    __syncthreads();
#pragma unroll 4
    for (int y = ty; y < kTile; y += 4) {
      const long long c = c0 + y, r = r0 + tx;  // output row = input column
      if (c < cols && r < rows) out[c * outStride + r] = tile[tx][y];
    }
    __syncthreads();
  }
}

// ---- register-block kernel ------------------------------------------------------------------------
struct TrParams {
  const char *in;
  char *out;
  long long rows, cols;
  long long inStrideBytes, outStrideBytes;
  unsigned int tilesX, tilesY;
  unsigned long long numTiles;
  int diagonalOrder;  // 0: row-major tile order, 1: diagonal tile order, 2: column-major tile order
};

// WR warps of the CTA along the input rows, 8 / WR along the input columns.  A warp covers 8 x 4 blocks with
// whole 128-byte lines on the store side (LOADFULL = false) or 4 x 8 blocks with whole lines on the load side
// (LOADFULL = true); every thread takes NB blocks, spaced so that the warp's short side grows to NB x 4 blocks.
template <int EB, int WR, bool LOADFULL, int NB>
__global__ void __launch_bounds__(256) transposeBlocksKernel(const __grid_constant__ TrParams p) {
  gridDependencyPrologue();
  using RB = RegBlock<EB>;
  using T = typename std::conditional<EB == 2, unsigned short, unsigned int>::type;
  constexpr int E = RB::kEdge;
  constexpr int WC = 8 / WR;
  constexpr int kWarpRows = (LOADFULL ? 4 * NB : 8) * E, kWarpCols = (LOADFULL ? 8 : 4 * NB) * E;
  constexpr int kTileRows = WR * kWarpRows, kTileCols = WC * kWarpCols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int li = LOADFULL ? (lane >> 3) : (lane & 7);  // block row of the thread's first block inside the warp tile
  const int lj = LOADFULL ? (lane & 7) : (lane >> 3);
  for (unsigned long long t = blockIdx.x; t < p.numTiles; t += gridDim.x) {
    unsigned int tx = static_cast<unsigned int>(t % p.tilesX);
    unsigned int ty = static_cast<unsigned int>(t / p.tilesX);
    // Optional diagonal order: tiles running at the same time then differ in tile row and tile column.
    if (p.diagonalOrder == 1) ty = (ty + tx) % p.tilesY;
    // Column-major order: neighbouring CTAs complete the same (short) output rows together.
    if (p.diagonalOrder == 2) {
      ty = static_cast<unsigned int>(t % p.tilesY);
      tx = static_cast<unsigned int>(t / p.tilesY);
    }
    const long long rw = static_cast<long long>(ty) * kTileRows + (warp / WC) * kWarpRows;
    const long long cw = static_cast<long long>(tx) * kTileCols + (warp % WC) * kWarpCols;
    long long r0[NB], c0[NB];
    bool whole[NB];
    uint4 a[NB][E];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      r0[b] = rw + static_cast<long long>(li + (LOADFULL ? 4 * b : 0)) * E;
      c0[b] = cw + static_cast<long long>(lj + (LOADFULL ? 0 : 4 * b)) * E;
      whole[b] = r0[b] + E <= p.rows && c0[b] + E <= p.cols;
      if (whole[b]) {
        const char *src = p.in + r0[b] * p.inStrideBytes + c0[b] * EB;
#pragma unroll
        for (int k = 0; k < E; ++k) a[b][k] = __ldcs(reinterpret_cast<const uint4 *>(src + k * p.inStrideBytes));
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      if (whole[b]) {
        uint4 o[E];
        RB::transpose(a[b], o);
        char *dst = p.out + c0[b] * p.outStrideBytes + r0[b] * EB;
#pragma unroll
        for (int k = 0; k < E; ++k) __stcs(reinterpret_cast<uint4 *>(dst + k * p.outStrideBytes), o[k]);
      } else {  // ragged edge: element by element
        for (int k = 0; k < E && r0[b] + k < p.rows; ++k)
          for (int e = 0; e < E && c0[b] + e < p.cols; ++e)
            *reinterpret_cast<T *>(p.out + (c0[b] + e) * p.outStrideBytes + (r0[b] + k) * EB) =
                *reinterpret_cast<const T *>(p.in + (r0[b] + k) * p.inStrideBytes + (c0[b] + e) * EB);
      }
    }
  }
}

template <int EB, bool LOADFULL, int NB>
void launchBlocksAs(const TrParams &base, int warpRows, long long rows, long long cols, int ctasPerSm, int smCount,
                    cudaStream_t stream) {
  constexpr int E = RegBlock<EB>::kEdge;
  TrParams p = base;
  const int wr = warpRows == 8 ? 8 : warpRows == 4 ? 4 : warpRows == 1 ? 1 : 2;
  const long long tileRows = static_cast<long long>(wr) * (LOADFULL ? 4 * NB : 8) * E;
  const long long tileCols = static_cast<long long>(8 / wr) * (LOADFULL ? 8 : 4 * NB) * E;
  const long long tilesX = (cols + tileCols - 1) / tileCols, tilesY = (rows + tileRows - 1) / tileRows;
  p.tilesX = static_cast<unsigned int>(tilesX);
  p.tilesY = static_cast<unsigned int>(tilesY);
  p.numTiles = static_cast<unsigned long long>(tilesX) * static_cast<unsigned long long>(tilesY);
  // one tile per CTA unless a persistent grid (SMs x ctasPerSm) is asked for
  unsigned long long want = ctasPerSm > 0 ? static_cast<unsigned long long>(smCount) * ctasPerSm : p.numTiles;
  const unsigned int grid = static_cast<unsigned int>(std::min<unsigned long long>(std::min(p.numTiles, want), 1u << 30));
  switch (wr) {
  case 8: launchDependent(transposeBlocksKernel<EB, 8, LOADFULL, NB>, grid, 256, 0, stream, p); break;
  case 4: launchDependent(transposeBlocksKernel<EB, 4, LOADFULL, NB>, grid, 256, 0, stream, p); break;
  case 1: launchDependent(transposeBlocksKernel<EB, 1, LOADFULL, NB>, grid, 256, 0, stream, p); break;
  default: launchDependent(transposeBlocksKernel<EB, 2, LOADFULL, NB>, grid, 256, 0, stream, p); break;
  }
}

template <int EB> void launchBlocks(const TrParams &p, int variant, int warpRows, long long rows, long long cols, int ctasPerSm,
                                    int smCount, cudaStream_t stream) {
  switch (variant) {
  case 1: launchBlocksAs<EB, false, 2>(p, warpRows, rows, cols, ctasPerSm, smCount, stream); break;
  case 2: launchBlocksAs<EB, true, 1>(p, warpRows, rows, cols, ctasPerSm, smCount, stream); break;
  case 3: launchBlocksAs<EB, true, 2>(p, warpRows, rows, cols, ctasPerSm, smCount, stream); break;
  default: launchBlocksAs<EB, false, 1>(p, warpRows, rows, cols, ctasPerSm, smCount, stream); break;
  }
}

int smCountOf() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

} // namespace

int launchTranspose(const TransposeLaunch &l, cudaStream_t stream, int *launched) {
  if (launched) *launched = 0;
  if (l.rows == 0 || l.cols == 0) return cudaSuccess;
  if (l.elemBytes != 2 && l.elemBytes != 4) return cudaErrorInvalidValue;
  const bool aligned = ((reinterpret_cast<uintptr_t>(l.in) | reinterpret_cast<uintptr_t>(l.out)) & 15u) == 0 &&
                       (l.inRowStride * l.elemBytes) % 16 == 0 && (l.outRowStride * l.elemBytes) % 16 == 0;
  // 16-bit elements: the copy-engine kernel (asked for with variant 4)
  if (aligned && !l.forceTileKernel && l.variant == 4 && transposeTmaApplies(l)) {
    const int rc = launchTransposeTma(l, smCountOf(), stream);
    if (launched && rc == cudaSuccess) *launched = 1;
    return rc;
  }
  if (aligned && !l.forceTileKernel) {
    TrParams p = {};
    p.in = static_cast<const char *>(l.in);
    p.out = static_cast<char *>(l.out);
    p.rows = l.rows;
    p.cols = l.cols;
    p.inStrideBytes = l.inRowStride * l.elemBytes;
    p.outStrideBytes = l.outRowStride * l.elemBytes;
    const int ctasPerSm = l.ctasPerSm > 0 ? l.ctasPerSm : 0;
    const int warpRows = l.warpRows > 0 ? l.warpRows : 2;
    p.diagonalOrder = l.diagonalOrder == 2 ? 2 : l.diagonalOrder ? 1 : 0;
    // Few input rows (a wide-and-low input, a tall-and-thin output whose rows are at most 4 KB): in row-major tile
    // order each output row would be finished by CTAs that run far apart in time, so the default walks the input
    // rows fastest there.
    if (l.diagonalOrder == 0 && l.rows * l.elemBytes <= 4096 && l.cols > l.rows) p.diagonalOrder = 2;
    if (l.elemBytes == 2) launchBlocks<2>(p, l.variant, warpRows, l.rows, l.cols, ctasPerSm, smCountOf(), stream);
    else launchBlocks<4>(p, l.variant, warpRows, l.rows, l.cols, ctasPerSm, smCountOf(), stream);
    if (launched) *launched = 1;
    return cudaGetLastError();
  }
  const long long tilesX = (l.cols + kTile - 1) / kTile;
  const long long tilesY = (l.rows + kTile - 1) / kTile;
  const unsigned long long numTiles = static_cast<unsigned long long>(tilesX) * tilesY;
  if (tilesX >= (1ll << 31)) return cudaErrorInvalidValue;
  const unsigned int grid = static_cast<unsigned int>(std::min<unsigned long long>(numTiles, 1u << 30));
  if (l.elemBytes == 2)
    launchDependent(transposeKernel<unsigned short>, grid, 256, 0, stream, static_cast<const unsigned short *>(l.in),
                                                              static_cast<unsigned short *>(l.out), l.rows, l.cols,
                                                              l.inRowStride, l.outRowStride,
                                                              static_cast<unsigned int>(tilesX), numTiles);
  else
    launchDependent(transposeKernel<unsigned int>, grid, 256, 0, stream, static_cast<const unsigned int *>(l.in),
                                                            static_cast<unsigned int *>(l.out), l.rows, l.cols,
                                                            l.inRowStride, l.outRowStride,
                                                            static_cast<unsigned int>(tilesX), numTiles);
  if (launched) *launched = 1;
  return cudaGetLastError();
}

} // namespace kernels
} // namespace afir
