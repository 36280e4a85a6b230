// Gather + elementwise fused groups.
//   axis 0, row gather:    out[i, j] = body(table[idx[i], j], views...)   -- the "embedding" form the
//       reference's structured-op marker tags as embedding_dim
//       (lib/Conversion/MarkStructuredOps/MarkStructuredOpsPass.cpp:54-139) and leaves unlowered
//       (lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:833-839);
//   axis 1, column gather: out[i, j] = body(table[i, idx[j]], views...)   -- the index_select form it
//       lowers (ComputeConversion.cpp:847-1273), pre-op -> extract -> post-op order per
//       lib/Conversion/FuseGatherElementwise/FuseGatherElementwisePass.cpp:190-274.
// A pre-op on the table commutes with the gather, so it is simply the first op of the body.
//
// HBM-bound.  Row gather: consecutive threads take consecutive 16-byte pieces of one gathered row,
// so a 512-byte row is one fully coalesced warp request; each thread keeps UNROLL rows in flight
// (indices first, then table pieces + the other views).  Column gather: each thread produces one
// 16-byte output vector from scalar loads of the (cache-resident) table row.
// Indices outside the table raise *status and leave the output untouched; nothing is clamped.
#include "kernels/ew_common.cuh"

#include <algorithm>

namespace afir {
namespace kernels {
namespace {

struct GaParams {
  const char *table;
  long long tableRows, tableCols, tableRowStride;
  const void *indices;
  int index64;
  const char *vbase[kMaxViews];
  long long rowStride[kMaxViews];
  int colStride[kMaxViews];
  int numViews;
  char *out;
  long long outRowStride;
  unsigned int vecPerRow;
  unsigned int totalVec;
  unsigned int numTiles;
  FastDiv divVpr;
  unsigned long long *status;
  BodyProgram prog;
};

__device__ __forceinline__ long long loadIndex(const void *idx, long long i, int is64) {
  return is64 ? __ldg(static_cast<const long long *>(idx) + i) : static_cast<long long>(__ldg(static_cast<const int *>(idx) + i));
}

template <class P> __device__ __forceinline__ void storeOne(void *p, P v);
template <> __device__ __forceinline__ void storeOne<PackF32>(void *p, PackF32 v) { *static_cast<float *>(p) = v.x; }
template <> __device__ __forceinline__ void storeOne<PackF16>(void *p, PackF16 v) {
  *static_cast<unsigned short *>(p) = static_cast<unsigned short>(v.bits() & 0xffffu);
}
template <> __device__ __forceinline__ void storeOne<PackBF16>(void *p, PackBF16 v) {
  *static_cast<unsigned short *>(p) = static_cast<unsigned short>(v.bits() & 0xffffu);
}

// ---- axis 0 ------------------------------------------------------------------------------------
template <class P, int BODY, int UNROLL, bool VECTOR>
__global__ void __launch_bounds__(512) gatherRowsKernel(const __grid_constant__ GaParams prm) {
  using B = Body<BODY>;
  constexpr int NV = B::kViews;
  constexpr int kElems = VECTOR ? Vec16<P>::kElems : 1;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
  const unsigned int tileVecs = blockDim.x * UNROLL;

  for (unsigned int tile = blockIdx.x; tile < prm.numTiles; tile += gridDim.x) {
    const unsigned int g0 = tile * tileVecs + threadIdx.x;
    unsigned int row[UNROLL], col[UNROLL];
    long long src[UNROLL];
    bool live[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const unsigned int g = g0 + u * blockDim.x;
      live[u] = g < prm.totalVec;
      row[u] = fastDivide(g, prm.divVpr);
      col[u] = g - row[u] * prm.vecPerRow;
      src[u] = live[u] ? loadIndex(prm.indices, row[u], prm.index64) : 0;
    }
    uint4 raw[UNROLL][NV];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (live[u] && (src[u] < 0 || src[u] >= prm.tableRows)) {
        if (col[u] == 0 && prm.status) atomicAdd(prm.status, 1ull);
        live[u] = false;
      }
      if (live[u]) {
        const char *t = prm.table + (src[u] * prm.tableRowStride + static_cast<long long>(col[u]) * kElems) * kElemBytes;
        if (VECTOR) raw[u][0] = loadStream16(t);
        else {
          const unsigned int s = P::splat(t).bits();
          raw[u][0] = make_uint4(s, s, s, s);
        }
#pragma unroll
        for (int k = 1; k < NV; ++k) {
          raw[u][k] = make_uint4(0u, 0u, 0u, 0u);
          if (k < prm.numViews) {
            const char *p = prm.vbase[k] + (static_cast<long long>(row[u]) * prm.rowStride[k] +
                                           static_cast<long long>(col[u]) * kElems * prm.colStride[k]) * kElemBytes;
            if (VECTOR && prm.colStride[k] == 1) raw[u][k] = prm.rowStride[k] == 0 ? loadKeep16(p) : loadStream16(p);
            else {
              const unsigned int s = P::splat(p).bits();
              raw[u][k] = make_uint4(s, s, s, s);
            }
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (!live[u]) continue;
      char *dst = prm.out + (static_cast<long long>(row[u]) * prm.outRowStride + static_cast<long long>(col[u]) * kElems) * kElemBytes;
      if (VECTOR) {
        Vec16<P> o;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          P v[NV];
#pragma unroll
          for (int k = 0; k < NV; ++k) {
            const unsigned int bits = q == 0 ? raw[u][k].x : q == 1 ? raw[u][k].y : q == 2 ? raw[u][k].z : raw[u][k].w;
            v[k] = P::fromBits(bits);
          }
          o.p[q] = B::template eval<P>(v, prm.prog);
        }
        storeStream16(dst, o.raw());
      } else {
        P v[NV];
#pragma unroll
        for (int k = 0; k < NV; ++k) v[k] = P::fromBits(raw[u][k].x);
        storeOne<P>(dst, B::template eval<P>(v, prm.prog));
      }
    }
  }
}

// ---- axis 1 ------------------------------------------------------------------------------------
// One output element per thread-iteration (the table accesses are scattered anyway; consecutive
// threads still write consecutive output elements).
template <class P, int BODY>
__global__ void __launch_bounds__(512) gatherColsKernel(const __grid_constant__ GaParams prm) {
  using B = Body<BODY>;
  constexpr int NV = B::kViews;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
  const unsigned int stride = gridDim.x * blockDim.x;
  for (unsigned int g = blockIdx.x * blockDim.x + threadIdx.x; g < prm.totalVec; g += stride) {
    const unsigned int row = fastDivide(g, prm.divVpr);
    const unsigned int col = g - row * prm.vecPerRow;
    const long long src = loadIndex(prm.indices, col, prm.index64);
    if (src < 0 || src >= prm.tableCols) {
      if (row == 0 && prm.status) atomicAdd(prm.status, 1ull);
      continue;
    }
    P v[NV];
    v[0] = P::splat(prm.table + (static_cast<long long>(row) * prm.tableRowStride + src) * kElemBytes);
#pragma unroll
    for (int k = 1; k < NV; ++k) {
      v[k] = v[0];
      if (k < prm.numViews)
        v[k] = P::splat(prm.vbase[k] + (static_cast<long long>(row) * prm.rowStride[k] +
                                        static_cast<long long>(col) * prm.colStride[k]) * kElemBytes);
    }
    storeOne<P>(prm.out + (static_cast<long long>(row) * prm.outRowStride + col) * kElemBytes,
                B::template eval<P>(v, prm.prog));
  }
}

using KernelFn = void (*)(const GaParams);

template <class P, int BODY> KernelFn pickRowsUnroll(int unroll, bool vector) {
  if (!vector) return gatherRowsKernel<P, BODY, 2, false>;
  return unroll >= 4 ? gatherRowsKernel<P, BODY, 4, true> : unroll >= 2 ? gatherRowsKernel<P, BODY, 2, true>
                                                                        : gatherRowsKernel<P, BODY, 1, true>;
}
template <class P> KernelFn pickRows(int body, int unroll, bool vector) {
  switch (body) {
  case kBodyCopy: return pickRowsUnroll<P, kBodyCopy>(unroll, vector);
  case kBodyMulAdd: return pickRowsUnroll<P, kBodyMulAdd>(unroll, vector);
  case kBodyAdd: return pickRowsUnroll<P, kBodyAdd>(unroll, vector);
  case kBodyMul: return pickRowsUnroll<P, kBodyMul>(unroll, vector);
  default: return pickRowsUnroll<P, kBodyInterpreted>(2, vector);
  }
}
template <class P> KernelFn pickCols(int body) {
  switch (body) {
  case kBodyCopy: return gatherColsKernel<P, kBodyCopy>;
  case kBodyReluAdd: return gatherColsKernel<P, kBodyReluAdd>;
  case kBodyAdd: return gatherColsKernel<P, kBodyAdd>;
  default: return gatherColsKernel<P, kBodyInterpreted>;
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

} // namespace

int launchGather(const GatherLaunch &l, cudaStream_t stream, int *launched) {
  if (launched) *launched = 0;
  if (l.rows == 0 || l.cols == 0) return cudaSuccess;
  if (l.numViews < 1 || l.numViews > kMaxViews) return cudaErrorInvalidValue;
  const int eb = elemBytes(l.elemType);
  const int vecElems = 16 / eb;

  GaParams p = {};
  p.table = static_cast<const char *>(l.table);
  p.tableRows = l.tableRows;
  p.tableCols = l.tableCols;
  p.tableRowStride = l.tableRowStride;
  p.indices = l.indices;
  p.index64 = l.indexType == kI64 ? 1 : 0;
  for (int k = 1; k < l.numViews; ++k) {
    p.vbase[k] = static_cast<const char *>(l.views[k].base);
    p.rowStride[k] = l.views[k].rowStride;
    p.colStride[k] = static_cast<int>(l.views[k].colStride);
  }
  p.numViews = l.numViews;
  p.out = static_cast<char *>(l.out);
  p.outRowStride = l.outRowStride;
  p.status = l.status;
  p.prog = l.body;

  int threads = l.ctaThreads > 0 ? l.ctaThreads : 128;
  threads = std::max(32, std::min(512, (threads / 32) * 32));
  const int body = matchBody(l.body, l.numViews);
  KernelFn fn;
  int64_t totalVec, numTiles;
  if (l.axis == 0) {
    bool vector = l.cols % vecElems == 0 && aligned16(l.table) && l.tableRowStride % vecElems == 0 &&
                  aligned16(l.out) && l.outRowStride % vecElems == 0;
    for (int k = 1; k < l.numViews && vector; ++k) {
      if (l.views[k].colStride == 1) vector = aligned16(l.views[k].base) && l.views[k].rowStride % vecElems == 0;
      else if (l.views[k].colStride != 0) vector = false;
    }
    int unroll = l.unroll > 0 ? l.unroll : 1;
    unroll = unroll >= 4 ? 4 : unroll >= 2 ? 2 : 1;
    if (!vector || body == kBodyInterpreted || (body != kBodyCopy && body != kBodyMulAdd && body != kBodyAdd && body != kBodyMul))
      unroll = 2;
    const int64_t vecPerRow = l.cols / (vector ? vecElems : 1);
    totalVec = l.rows * vecPerRow;
    if (totalVec >= (1ll << 32) - (1 << 20) || vecPerRow >= (1ll << 31)) return cudaErrorInvalidValue;
    p.vecPerRow = static_cast<unsigned int>(vecPerRow);
    fn = l.elemType == kF32 ? pickRows<PackF32>(body, unroll, vector)
         : l.elemType == kF16 ? pickRows<PackF16>(body, unroll, vector)
                              : pickRows<PackBF16>(body, unroll, vector);
    const int64_t tileVecs = static_cast<int64_t>(threads) * unroll;
    numTiles = (totalVec + tileVecs - 1) / tileVecs;
  } else {
    totalVec = l.rows * l.cols;
    if (totalVec >= (1ll << 32) - (1 << 20) || l.cols >= (1ll << 31)) return cudaErrorInvalidValue;
    p.vecPerRow = static_cast<unsigned int>(l.cols);
    fn = l.elemType == kF32 ? pickCols<PackF32>(body) : l.elemType == kF16 ? pickCols<PackF16>(body) : pickCols<PackBF16>(body);
    numTiles = (totalVec + threads - 1) / threads;
  }
  p.totalVec = static_cast<unsigned int>(totalVec);
  p.numTiles = static_cast<unsigned int>(numTiles);
  p.divVpr = makeFastDiv(p.vecPerRow);
  int64_t grid = l.gridBlocks > 0 ? l.gridBlocks : numTiles;
  grid = std::max<int64_t>(1, std::min<int64_t>(grid, numTiles));
  fn<<<static_cast<unsigned int>(grid), threads, 0, stream>>>(p);
  if (launched) *launched = 1;
  return cudaGetLastError();
}

} // namespace kernels
} // namespace afir
