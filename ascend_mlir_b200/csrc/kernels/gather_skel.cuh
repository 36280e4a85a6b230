// Device side of the row-gather kernel (out[i, j] = body(table[idx[i], j], views...)): the launch record and the
// tile loop as a function template over the fused body.  The prebuilt kernels instantiate it with the straight-line
// bodies and the interpreter; a kernel generated for one fused group instantiates it with that group's own body.
// (Also compiled at run time by NVRTC: no host headers here.)
#pragma once

#include "kernels/ew_common.cuh"

namespace afir {
namespace kernels {

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
  FastDiv divVpr;
  unsigned long long *status;
  BodyProgram prog;
  // SHARDED kernels: the table's rows are split into contiguous shards of rowsPerShard rows, shard s at
  // shardBase[s], which may be another GPU's memory (peer-mapped; read with plain loads over NVLink)
  const char *shardBase[kMaxTableShards];
  long long rowsPerShard;
  FastDiv divRowsPerShard;  // valid when the table has fewer than 2^32 rows
};

__device__ __forceinline__ long long loadIndex(const void *idx, long long i, int is64) {
  return is64 ? __ldg(static_cast<const long long *>(idx) + i) : static_cast<long long>(__ldg(static_cast<const int *>(idx) + i));
}

template <class P> __device__ __forceinline__ void storeOne(void *p, P v);
template <> __device__ __forceinline__ void storeOne<PackF32>(void *p, PackF32 v) { *static_cast<float *>(p) = v.x; }
#ifdef AFIR_HAVE_F16
template <> __device__ __forceinline__ void storeOne<PackF16>(void *p, PackF16 v) {
  *static_cast<unsigned short *>(p) = static_cast<unsigned short>(v.bits() & 0xffffu);
}
#endif
#ifdef AFIR_HAVE_BF16
template <> __device__ __forceinline__ void storeOne<PackBF16>(void *p, PackBF16 v) {
  *static_cast<unsigned short *>(p) = static_cast<unsigned short>(v.bits() & 0xffffu);
}
#endif

// ---- axis 0 ------------------------------------------------------------------------------------
template <class P, class B, int UNROLL, bool VECTOR, bool SHARDED = false, bool PLAINDIV = false>
__device__ __forceinline__ void gatherRowsTiles(const GaParams &prm) {
  constexpr int NV = B::kViews;
  constexpr int kElems = VECTOR ? Vec16<P>::kElems : 1;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
  const unsigned int tileVecs = blockDim.x * UNROLL;

  // Tiles are walked until one starts past the last vector: no tile count (and no division to get it) is needed.
  for (unsigned int tile = blockIdx.x;; tile += gridDim.x) {
    const unsigned long long tileBase = static_cast<unsigned long long>(tile) * tileVecs;
    if (tileBase >= prm.totalVec) break;
    const unsigned int g0 = static_cast<unsigned int>(tileBase) + threadIdx.x;
    unsigned int row[UNROLL], col[UNROLL];
    long long src[UNROLL];
    bool live[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const unsigned int g = g0 + u * blockDim.x;
      live[u] = g < prm.totalVec;
      row[u] = PLAINDIV ? g / prm.vecPerRow : fastDivide(g, prm.divVpr);
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
        const char *t;
        if (SHARDED) {
          const unsigned int shard = fastDivide(static_cast<unsigned int>(src[u]), prm.divRowsPerShard);
          const long long local = src[u] - static_cast<long long>(shard) * prm.rowsPerShard;
          t = prm.shardBase[shard] + (local * prm.tableRowStride + static_cast<long long>(col[u]) * kElems) * kElemBytes;
        } else {
          t = prm.table + (src[u] * prm.tableRowStride + static_cast<long long>(col[u]) * kElems) * kElemBytes;
        }
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
      if (VECTOR && B::kInterpreted) {
        storeStream16(dst, evalVector16<B, P, NV>(raw[u], prm.prog));
      } else if (VECTOR) {
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

} // namespace kernels
} // namespace afir
