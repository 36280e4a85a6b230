// 2-D transpose out[c, r] = in[r, c] (permutation generics,
// lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:1275-1290).
// HBM-bound: a 64x64 tile is read with coalesced rows into padded shared memory and written back
// with coalesced rows of the transposed tile, so both global sides move full 128-byte lines.
#include <cuda_runtime.h>

#include <algorithm>

#include "kernels/kernels.h"

namespace afir {
namespace kernels {
namespace {

constexpr int kTile = 64;

template <typename T>
__global__ void __launch_bounds__(256) transposeKernel(const T *__restrict__ in, T *__restrict__ out, long long rows,
                                                       long long cols, long long inStride, long long outStride,
                                                       unsigned int tilesX, unsigned long long numTiles) {
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

} // namespace

int launchTranspose(const TransposeLaunch &l, cudaStream_t stream, int *launched) {
  if (launched) *launched = 0;
  if (l.rows == 0 || l.cols == 0) return cudaSuccess;
  if (l.elemBytes != 2 && l.elemBytes != 4) return cudaErrorInvalidValue;
  const long long tilesX = (l.cols + kTile - 1) / kTile;
  const long long tilesY = (l.rows + kTile - 1) / kTile;
  const unsigned long long numTiles = static_cast<unsigned long long>(tilesX) * tilesY;
  if (tilesX >= (1ll << 31)) return cudaErrorInvalidValue;
  const unsigned int grid = static_cast<unsigned int>(std::min<unsigned long long>(numTiles, 1u << 30));
  if (l.elemBytes == 2)
    transposeKernel<unsigned short><<<grid, 256, 0, stream>>>(static_cast<const unsigned short *>(l.in),
                                                              static_cast<unsigned short *>(l.out), l.rows, l.cols,
                                                              l.inRowStride, l.outRowStride,
                                                              static_cast<unsigned int>(tilesX), numTiles);
  else
    transposeKernel<unsigned int><<<grid, 256, 0, stream>>>(static_cast<const unsigned int *>(l.in),
                                                            static_cast<unsigned int *>(l.out), l.rows, l.cols,
                                                            l.inRowStride, l.outRowStride,
                                                            static_cast<unsigned int>(tilesX), numTiles);
  if (launched) *launched = 1;
  return cudaGetLastError();
}

} // namespace kernels
} // namespace afir
