// Device side of the elementwise / broadcast / split / concat kernels: the launch record and the tile loop, as a
// function template over the fused body.  The prebuilt kernels instantiate it with the straight-line bodies and
// the interpreter; a kernel generated for one fused group instantiates it with that group's own body.
// (Also compiled at run time by NVRTC: no host headers here.)
#pragma once

#include "kernels/ew_common.cuh"

namespace afir {
namespace kernels {

struct EwParams {
  const char *vbase[kMaxViews];
  long long vs0[kMaxViews], vs1[kMaxViews], vs2[kMaxViews];
  char *obase;
  long long os0, os1;
  unsigned int vecPerRow;  // vectors (or elements, scalar variant) along the inner dim
  unsigned int d1;
  unsigned int totalVec;
  unsigned int numTiles;
  FastDiv divVpr, divD1;
  int flat;  // inner dim is the whole domain: skip the row arithmetic
  int numViews;
  BodyProgram prog;
  long long vOuterBytes[kMaxViews];  // OUTER kernels: byte offset per blockIdx.y, per view and for the output
  long long oOuterBytes;
};

template <class P> __device__ __forceinline__ void storeScalar(void *p, P v);
template <> __device__ __forceinline__ void storeScalar<PackF32>(void *p, PackF32 v) {
  *reinterpret_cast<float *>(p) = v.x;
}
#ifdef AFIR_HAVE_F16
template <> __device__ __forceinline__ void storeScalar<PackF16>(void *p, PackF16 v) {
  *reinterpret_cast<unsigned short *>(p) = static_cast<unsigned short>(v.bits() & 0xffffu);
}
#endif
#ifdef AFIR_HAVE_BF16
template <> __device__ __forceinline__ void storeScalar<PackBF16>(void *p, PackBF16 v) {
  *reinterpret_cast<unsigned short *>(p) = static_cast<unsigned short>(v.bits() & 0xffffu);
}
#endif
template <> __device__ __forceinline__ void storeScalar<PackI32>(void *p, PackI32 v) { *reinterpret_cast<int *>(p) = v.x; }
template <> __device__ __forceinline__ void storeScalar<PackI16>(void *p, PackI16 v) {
  *reinterpret_cast<unsigned short *>(p) = static_cast<unsigned short>(v.bits() & 0xffffu);
}

// PLAINDIV: index arithmetic with `/` instead of the precomputed multiply-shift (generated kernels: their
// extents are compile-time literals more often than not, and they have no host to prepare the magic numbers).
template <class P, class B, int UNROLL, bool VECTOR, bool OUTER = false, bool PLAINDIV = false>
__device__ __forceinline__ void elementwiseTiles(const EwParams &prm) {
  constexpr int NV = B::kViews;
  constexpr int kElems = VECTOR ? Vec16<P>::kElems : 1;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
  const unsigned int tileVecs = blockDim.x * UNROLL;

  for (unsigned int tile = blockIdx.x; tile < prm.numTiles; tile += gridDim.x) {
    const unsigned int g0 = tile * tileVecs + threadIdx.x;
    uint4 raw[UNROLL][NV];
    long long ooff[UNROLL];
    bool live[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const unsigned int g = g0 + u * blockDim.x;
      live[u] = g < prm.totalVec;
      unsigned int col = g, i0 = 0, i1 = 0;
      if (!prm.flat) {
        const unsigned int row = PLAINDIV ? g / prm.vecPerRow : fastDivide(g, prm.divVpr);
        col = g - row * prm.vecPerRow;
        i0 = PLAINDIV ? row / prm.d1 : fastDivide(row, prm.divD1);
        i1 = row - i0 * prm.d1;
      }
      ooff[u] = (static_cast<long long>(i0) * prm.os0 + static_cast<long long>(i1) * prm.os1 +
                 static_cast<long long>(col) * kElems) * kElemBytes + (OUTER ? blockIdx.y * prm.oOuterBytes : 0ll);
      if (live[u]) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          if (k < prm.numViews) {
            const long long e = static_cast<long long>(i0) * prm.vs0[k] + static_cast<long long>(i1) * prm.vs1[k] +
                                static_cast<long long>(col) * kElems * prm.vs2[k];
            const char *src = prm.vbase[k] + e * kElemBytes + (OUTER ? blockIdx.y * prm.vOuterBytes[k] : 0ll);
            if (VECTOR && prm.vs2[k] == 1) {
              raw[u][k] = loadStream16(src);
            } else {
              const unsigned int s = P::splat(src).bits();
              raw[u][k] = make_uint4(s, s, s, s);
            }
          } else {
            raw[u][k] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (!live[u]) continue;
      if (VECTOR && B::kInterpreted) {
        storeStream16(prm.obase + ooff[u], evalVector16<B, P, NV>(raw[u], prm.prog));
      } else if (VECTOR) {
        Vec16<P> in[NV];
#pragma unroll
        for (int k = 0; k < NV; ++k) in[k] = Vec16<P>::fromRaw(raw[u][k]);
        Vec16<P> out;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          P v[NV];
#pragma unroll
          for (int k = 0; k < NV; ++k) v[k] = in[k].p[q];
          out.p[q] = B::template eval<P>(v, prm.prog);
        }
        storeStream16(prm.obase + ooff[u], out.raw());
      } else {
        P v[NV];
#pragma unroll
        for (int k = 0; k < NV; ++k) v[k] = P::fromBits(raw[u][k].x);
        storeScalar<P>(prm.obase + ooff[u], B::template eval<P>(v, prm.prog));
      }
    }
  }
}

} // namespace kernels
} // namespace afir
