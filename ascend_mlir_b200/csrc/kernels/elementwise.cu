// Elementwise / broadcast / split / concat fused groups (the all-parallel linalg.generic class the
// reference lowers in lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:750-1624, with split and
// concat folded into view offsets as lib/Conversion/Passes.td:72-102 does for concat).
//
// HBM-bound: every thread keeps UNROLL independent 16-byte loads per view in flight, inputs read
// once are loaded with the streaming (evict-first) policy, broadcast operands through the read-only
// path.  No shared memory: there is no reuse to stage.  Arithmetic rounds after every op.
#include "kernels/elementwise_blocks_skel.cuh"
#include "kernels/elementwise_skel.cuh"
#include "kernels/launch_util.h"
#include "kernels/reg_block.cuh"

#include <algorithm>
#include <mutex>

namespace afir {
namespace kernels {
namespace {

template <class P, int BODY, int UNROLL, bool VECTOR, bool OUTER = false>
__global__ void __launch_bounds__(512) elementwiseKernel(const __grid_constant__ EwParams prm) {
  gridDependencyPrologue();
  elementwiseTiles<P, Body<BODY>, UNROLL, VECTOR, OUTER>(prm);
}

using KernelFn = void (*)(const EwParams);

template <class P, int BODY> KernelFn pickUnroll(int unroll) {
  switch (unroll) {
  case 1: return elementwiseKernel<P, BODY, 1, true>;
  case 2: return elementwiseKernel<P, BODY, 2, true>;
  default: return elementwiseKernel<P, BODY, 4, true>;
  }
}

template <class P> KernelFn pickVector(int body, int unroll) {
  switch (body) {
  case kBodyCopy: return pickUnroll<P, kBodyCopy>(unroll);
  case kBodyAdd: return pickUnroll<P, kBodyAdd>(unroll);
  case kBodyMul: return pickUnroll<P, kBodyMul>(unroll);
  case kBodyAddMulRhs: return pickUnroll<P, kBodyAddMulRhs>(unroll);
  case kBodyAddMul: return pickUnroll<P, kBodyAddMul>(unroll);
  case kBodyMulAdd: return pickUnroll<P, kBodyMulAdd>(unroll);
  case kBodyReluAdd: return pickUnroll<P, kBodyReluAdd>(unroll);
  case kBodyReluAddMul: return pickUnroll<P, kBodyReluAddMul>(unroll);
  case kBodyRelu: return pickUnroll<P, kBodyRelu>(unroll);
  default: return elementwiseKernel<P, kBodyInterpreted, 2, true>;
  }
}

template <class P> KernelFn pickScalar() { return elementwiseKernel<P, kBodyInterpreted, 2, false>; }

// Kernels that take one more outer dim from blockIdx.y: the copy body (permutations) and the interpreted body.
template <class P> KernelFn pickOuter(int body, bool vector) {
  if (!vector) return elementwiseKernel<P, kBodyInterpreted, 2, false, true>;
  if (body == kBodyCopy) return elementwiseKernel<P, kBodyCopy, 2, true, true>;
  return elementwiseKernel<P, kBodyInterpreted, 2, true, true>;
}
template <class P> KernelFn pickOuterInteger(bool vector) {
  return vector ? elementwiseKernel<P, kBodyInterpreted, 2, true, true> : elementwiseKernel<P, kBodyInterpreted, 2, false, true>;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- block variant: groups with an operand read through a transposed view (kernels/elementwise_blocks_skel.cuh) ----
template <class P, int BODY, int NVL>
__global__ void __launch_bounds__(256) elementwiseBlocksKernel(const __grid_constant__ EbParams prm) {
  gridDependencyPrologue();
  elementwiseBlocksTiles<P, Body<BODY>, NVL>(prm);
}

using BlocksFn = void (*)(const EbParams);
template <class P> BlocksFn pickBlocks(int body, int numViews) {
  switch (body) {
  case kBodyCopy: return elementwiseBlocksKernel<P, kBodyCopy, 1>;
  case kBodyAdd: return elementwiseBlocksKernel<P, kBodyAdd, 2>;
  case kBodyMul: return elementwiseBlocksKernel<P, kBodyMul, 2>;
  case kBodyAddMul: return elementwiseBlocksKernel<P, kBodyAddMul, 3>;
  case kBodyMulAdd: return elementwiseBlocksKernel<P, kBodyMulAdd, 3>;
  case kBodyReluAdd: return elementwiseBlocksKernel<P, kBodyReluAdd, 2>;
  default: return numViews <= 3 ? elementwiseBlocksKernel<P, kBodyInterpreted, 3> : nullptr;
  }
}

// Launches the block variant when the group has a transposed view and everything is aligned for it.
// Returns false (nothing launched) when the group does not qualify.
bool tryLaunchBlocks(const ElementwiseLaunch &l, cudaStream_t stream, cudaError_t &err) {
  const int eb = elemBytes(l.elemType);
  const int E = 16 / eb;
  bool anyTransposed = false;
  EbParams p = {};
  if (!aligned16(l.outBase) || l.outStride[0] % E || l.outStride[1] % E) return false;
  for (int k = 0; k < l.numViews; ++k) {
    const ViewAccess &v = l.views[k];
    p.vbase[k] = static_cast<const char *>(v.base);
    p.s0[k] = v.stride[0];
    p.s1[k] = v.stride[1];
    p.s2[k] = v.stride[2];
    if (v.stride[2] == 1) {
      p.kind[k] = kViewRowMajor;
      if (!aligned16(v.base) || v.stride[0] % E || v.stride[1] % E) return false;
    } else if (v.stride[2] == 0) {
      p.kind[k] = kViewInnerBroadcast;
    } else if (v.stride[1] == 1) {
      p.kind[k] = kViewTransposed;
      anyTransposed = true;
      if (!aligned16(v.base) || v.stride[0] % E || v.stride[2] % E) return false;
    } else {
      return false;
    }
  }
  if (!anyTransposed) return false;
  int body = matchBody(l.body, l.numViews);
  if (body != kBodyCopy && body != kBodyAdd && body != kBodyMul && body != kBodyAddMul && body != kBodyMulAdd && body != kBodyReluAdd)
    body = kBodyInterpreted;
  BlocksFn fn = nullptr;
  if (l.elemType == kInt32 || l.elemType == kInt16) {  // integers: the interpreted body only
    if (l.numViews <= 3) fn = l.elemType == kInt32 ? elementwiseBlocksKernel<PackI32, kBodyInterpreted, 3> : elementwiseBlocksKernel<PackI16, kBodyInterpreted, 3>;
  } else {
    fn = l.elemType == kF32 ? pickBlocks<PackF32>(body, l.numViews)
         : l.elemType == kF16 ? pickBlocks<PackF16>(body, l.numViews)
                              : pickBlocks<PackBF16>(body, l.numViews);
  }
  if (!fn) return false;
  const long long tileRows = 2 * 4 * E, tileCols = 4 * 8 * E;
  const long long tilesX = (l.dims[2] + tileCols - 1) / tileCols, tilesY = (l.dims[1] + tileRows - 1) / tileRows;
  if (tilesX >= (1ll << 31) || tilesY >= (1ll << 31)) return false;
  p.numViews = l.numViews;
  p.obase = static_cast<char *>(l.outBase);
  p.os0 = l.outStride[0];
  p.os1 = l.outStride[1];
  p.d1 = l.dims[1];
  p.d2 = l.dims[2];
  p.tilesX = static_cast<unsigned int>(tilesX);
  p.tilesY = static_cast<unsigned int>(tilesY);
  p.numTiles = static_cast<unsigned long long>(l.dims[0]) * tilesX * tilesY;
  p.prog = l.body;
  unsigned long long grid = l.gridBlocks > 0 ? static_cast<unsigned long long>(l.gridBlocks) : p.numTiles;
  grid = std::max<unsigned long long>(1, std::min<unsigned long long>(std::min(grid, p.numTiles), 1u << 30));
  launchDependent(fn, static_cast<unsigned int>(grid), 256, 0, stream, p);
  err = cudaGetLastError();
  return true;
}

} // namespace

int deviceSmCount(int device) {
  static std::mutex mu;
  static int cached[64];
  std::lock_guard<std::mutex> lock(mu);
  if (device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cached[device] = n;
  }
  return cached[device];
}

const char *cudaErrorText(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }

int launchElementwise(const ElementwiseLaunch &given, cudaStream_t stream, int *launched) {
  if (launched) *launched = 0;
  const int64_t total = given.dims[0] * given.dims[1] * given.dims[2];
  if (total == 0) return cudaSuccess;
  if (given.numViews < 1 || given.numViews > kMaxViews || given.outStride[2] != 1) return cudaErrorInvalidValue;

  // One more outer dim: as the grid's second dimension when every view is contiguous or constant along the inner
  // dim (the 16-byte kernel or its element twin runs, nothing else), otherwise one launch per outer index.
  bool outerInGrid = false;
  if (given.outerCount > 1) {
    outerInGrid = given.outerCount <= 65535;
    for (int k = 0; k < given.numViews; ++k)
      if (given.views[k].stride[2] != 0 && given.views[k].stride[2] != 1) outerInGrid = false;
    if (!outerInGrid) {
      const int ebytes = elemBytes(given.elemType);
      ElementwiseLaunch one = given;
      one.outerCount = 1;
      int total = 0;
      for (int64_t o = 0; o < given.outerCount; ++o) {
        for (int k = 0; k < given.numViews; ++k)
          one.views[k].base = static_cast<const char *>(given.views[k].base) + o * given.viewOuterStride[k] * ebytes;
        one.outBase = static_cast<char *>(given.outBase) + o * given.outOuterStride * ebytes;
        int n = 0;
        const int rc = launchElementwise(one, stream, &n);
        total += n;
        if (launched) *launched = total;
        if (rc != cudaSuccess) return rc;
      }
      return cudaSuccess;
    }
  }

  // The block variant wants a transposed view contiguous along the MIDDLE dim.  All three dims are parallel, so
  // when such a view is contiguous along the outer dim instead (out[i,j,k] = in[k,j,i]) the two outer dims
  // trade places: same elements, same addresses, another walking order.
  ElementwiseLaunch l = given;
  if (!l.forceElementAccess) {
    bool swapHelps = false, swapHurts = false;
    for (int k = 0; k < l.numViews; ++k) {
      const ViewAccess &v = l.views[k];
      if (v.stride[2] == 0 || v.stride[2] == 1) continue;
      if (v.stride[1] != 1 && v.stride[0] == 1 && l.dims[0] > 1) swapHelps = true;
      if (v.stride[1] == 1) swapHurts = true;
    }
    if (swapHelps && !swapHurts) {
      std::swap(l.dims[0], l.dims[1]);
      std::swap(l.outStride[0], l.outStride[1]);
      for (int k = 0; k < l.numViews; ++k) std::swap(l.views[k].stride[0], l.views[k].stride[1]);
    }
  }

  const int eb = elemBytes(l.elemType);
  const int vecElems = 16 / eb;
  // A bare copy of one transposed 2-D view is a transpose: out[r, c] = in[c, r] with `in` c-major.
  if (!l.forceElementAccess && l.numViews == 1 && l.dims[0] == 1 && l.views[0].stride[1] == 1 && l.views[0].stride[2] > 1 &&
      (eb == 2 || eb == 4) && matchBody(l.body, 1) == kBodyCopy) {
    TransposeLaunch t = {};
    t.elemBytes = eb;
    t.rows = l.dims[2];  // shape of the input as stored: [dims[2], dims[1]]
    t.cols = l.dims[1];
    t.in = l.views[0].base;
    t.inRowStride = l.views[0].stride[2];
    t.out = l.outBase;
    t.outRowStride = l.outStride[1];
    return launchTranspose(t, stream, launched);  // (variant 0: the register-block kernel, which waits for nothing)
  }
  {  // a transposed operand: the block variant keeps every access 16 bytes wide
    cudaError_t berr = cudaSuccess;
    if (!l.forceElementAccess && tryLaunchBlocks(l, stream, berr)) {
      if (launched) *launched = 1;
      return berr;
    }
  }
  // The 16-byte path needs every contiguous view (and the output) to start on a 16-byte boundary
  // with all outer strides and the inner extent multiples of the vector; inner strides 0 or 1.
  bool vector = l.dims[2] % vecElems == 0 && aligned16(l.outBase) && l.outStride[0] % vecElems == 0 &&
                l.outStride[1] % vecElems == 0;
  for (int k = 0; k < l.numViews && vector; ++k) {
    const ViewAccess &v = l.views[k];
    if (v.stride[2] == 1)
      vector = aligned16(v.base) && v.stride[0] % vecElems == 0 && v.stride[1] % vecElems == 0 &&
               (!outerInGrid || l.viewOuterStride[k] % vecElems == 0);
    else if (v.stride[2] != 0)
      vector = false;
  }
  if (outerInGrid && l.outOuterStride % vecElems != 0) vector = false;
  const int perVec = vector ? vecElems : 1;
  const int64_t vecPerRow = l.dims[2] / perVec;
  const int64_t totalVec = l.dims[0] * l.dims[1] * vecPerRow;
  if (totalVec >= (1ll << 32) - (1 << 20) || l.dims[1] >= (1ll << 31) || vecPerRow >= (1ll << 31))
    return cudaErrorInvalidValue;

  EwParams p = {};
  for (int k = 0; k < l.numViews; ++k) {
    p.vbase[k] = static_cast<const char *>(l.views[k].base);
    p.vs0[k] = l.views[k].stride[0];
    p.vs1[k] = l.views[k].stride[1];
    p.vs2[k] = l.views[k].stride[2];
  }
  p.obase = static_cast<char *>(l.outBase);
  p.os0 = l.outStride[0];
  p.os1 = l.outStride[1];
  p.vecPerRow = static_cast<unsigned int>(vecPerRow);
  p.d1 = static_cast<unsigned int>(l.dims[1]);
  p.totalVec = static_cast<unsigned int>(totalVec);
  p.divVpr = makeFastDiv(p.vecPerRow);
  p.divD1 = makeFastDiv(p.d1);
  p.flat = (l.dims[0] == 1 && l.dims[1] == 1) ? 1 : 0;
  p.numViews = l.numViews;
  p.prog = l.body;
  if (outerInGrid) {
    for (int k = 0; k < l.numViews; ++k) p.vOuterBytes[k] = l.viewOuterStride[k] * eb;
    p.oOuterBytes = l.outOuterStride * eb;
  }

  int threads = l.ctaThreads > 0 ? l.ctaThreads : 128;
  threads = std::max(32, std::min(512, (threads / 32) * 32));
  int unroll = l.unroll > 0 ? l.unroll : 2;
  unroll = unroll >= 4 ? 4 : (unroll >= 2 ? 2 : 1);
  const int body = vector ? matchBody(l.body, l.numViews) : kBodyInterpreted;
  if (!vector || body == kBodyInterpreted) unroll = 2;

  KernelFn fn = nullptr;
  if (l.elemType == kInt32 || l.elemType == kInt16) {
    // integer groups run the interpreted body (no specialised chains: they are not on a measured path)
    unroll = 2;
    if (l.elemType == kInt32) fn = vector ? elementwiseKernel<PackI32, kBodyInterpreted, 2, true> : pickScalar<PackI32>();
    else fn = vector ? elementwiseKernel<PackI16, kBodyInterpreted, 2, true> : pickScalar<PackI16>();
  } else if (vector) {
    fn = l.elemType == kF32 ? pickVector<PackF32>(body, unroll)
         : l.elemType == kF16 ? pickVector<PackF16>(body, unroll)
                              : pickVector<PackBF16>(body, unroll);
  } else {
    fn = l.elemType == kF32 ? pickScalar<PackF32>() : l.elemType == kF16 ? pickScalar<PackF16>() : pickScalar<PackBF16>();
  }

  if (outerInGrid) {
    unroll = 2;
    if (l.elemType == kInt32) fn = pickOuterInteger<PackI32>(vector);
    else if (l.elemType == kInt16) fn = pickOuterInteger<PackI16>(vector);
    else fn = l.elemType == kF32 ? pickOuter<PackF32>(body, vector) : l.elemType == kF16 ? pickOuter<PackF16>(body, vector)
                                                                                         : pickOuter<PackBF16>(body, vector);
  }

  const int64_t tileVecs = static_cast<int64_t>(threads) * unroll;
  const int64_t numTiles = (totalVec + tileVecs - 1) / tileVecs;
  p.numTiles = static_cast<unsigned int>(numTiles);
  int64_t grid = l.gridBlocks > 0 ? l.gridBlocks : numTiles;
  grid = std::max<int64_t>(1, std::min<int64_t>(grid, numTiles));
  const dim3 blocks(static_cast<unsigned int>(grid), outerInGrid ? static_cast<unsigned int>(l.outerCount) : 1u);
  launchDependent(fn, blocks, threads, 0, stream, p);
  if (launched) *launched = 1;
  return cudaGetLastError();
}

} // namespace kernels
} // namespace afir
