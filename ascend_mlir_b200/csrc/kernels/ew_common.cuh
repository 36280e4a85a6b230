// Shared device-side pieces of the bandwidth-bound fused-group kernels: 16-byte vector packs per
// element type, per-op-rounded arithmetic, the specialised body functors and the body interpreter.
//
// This file and the *_skel.cuh files beside it are also compiled at run time: the kernel generator embeds them
// and hands them to NVRTC as the headers of every generated kernel, so they use no host header.  A generated
// translation unit defines AFIR_CG_F16 / AFIR_CG_BF16 when its group computes in that type; the 16-bit packs
// (and the CUDA headers they need) are left out otherwise, which keeps an f32 or integer kernel's compile short.
#pragma once

#if !defined(__CUDACC_RTC__) || defined(AFIR_CG_F16)
#define AFIR_HAVE_F16 1
#include <cuda_fp16.h>
#endif
#if !defined(__CUDACC_RTC__) || defined(AFIR_CG_BF16)
#define AFIR_HAVE_BF16 1
#include <cuda_bf16.h>
#endif
#ifndef __CUDACC_RTC__
#include <cuda_runtime.h>
#endif

#include "kernels/grid_dependency.cuh"
#include "kernels/kernels.h"

namespace afir {
namespace kernels {

// ---- 32-bit division by a launch-time constant ------------------------------------------------
struct FastDiv {
  unsigned int magic;
  unsigned int shift;
  unsigned int divisor;
};
__host__ __device__ inline FastDiv makeFastDiv(unsigned int d) {
  FastDiv f;
  f.divisor = d;
  unsigned int s = 0;
  while ((1ull << s) < d) ++s;
  f.shift = s;
  f.magic = static_cast<unsigned int>(((1ull << 32) * ((1ull << s) - d)) / d + 1);
  return f;
}
__device__ __forceinline__ unsigned int fastDivide(unsigned int n, const FastDiv &f) {
  unsigned long long t = static_cast<unsigned long long>(__umulhi(n, f.magic)) + n;
  return static_cast<unsigned int>(t >> f.shift);
}

// ---- streaming 16-byte global access ----------------------------------------------------------
__device__ __forceinline__ uint4 loadStream16(const void *p) {
  return __ldcs(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ uint4 loadKeep16(const void *p) {
  return __ldg(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ void storeStream16(void *p, const uint4 &v) {
  __stcs(reinterpret_cast<uint4 *>(p), v);
}

// ---- packs: one 32-bit register worth of elements ----------------------------------------------
// arith.maximumf / minimumf propagate NaN and order -0 < +0: max.NaN / min.NaN do exactly that.
struct PackF32 {
  using Scalar = float;
  static constexpr int kLanes = 1;
  float x;
  __device__ __forceinline__ static PackF32 fromBits(unsigned int u) { return {__uint_as_float(u)}; }
  __device__ __forceinline__ unsigned int bits() const { return __float_as_uint(x); }
  __device__ __forceinline__ static PackF32 splat(const void *p) {
    return {__ldg(reinterpret_cast<const float *>(p))};
  }
  __device__ __forceinline__ static PackF32 constant(float c) { return {c}; }
  __device__ __forceinline__ static PackF32 constantOf(const BodySrc &s) { return constant(s.value); }
  __device__ __forceinline__ static PackF32 add(PackF32 a, PackF32 b) { return {__fadd_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackF32 sub(PackF32 a, PackF32 b) { return {__fsub_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackF32 mul(PackF32 a, PackF32 b) { return {__fmul_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackF32 div(PackF32 a, PackF32 b) { return {__fdiv_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackF32 max(PackF32 a, PackF32 b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a.x), "f"(b.x));
    return {r};
  }
  __device__ __forceinline__ static PackF32 min(PackF32 a, PackF32 b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a.x), "f"(b.x));
    return {r};
  }
  __device__ __forceinline__ float lane(int) const { return x; }
  __device__ __forceinline__ static unsigned short scalarBits(float) { return 0; }
};

#ifdef AFIR_HAVE_F16
struct PackF16 {
  using Scalar = __half;
  static constexpr int kLanes = 2;
  __half2 x;
  __device__ __forceinline__ static PackF16 fromBits(unsigned int u) {
    PackF16 p;
    p.x = *reinterpret_cast<__half2 *>(&u);
    return p;
  }
  __device__ __forceinline__ unsigned int bits() const { return *reinterpret_cast<const unsigned int *>(&x); }
  __device__ __forceinline__ static PackF16 splat(const void *p) {
    unsigned short u = __ldg(reinterpret_cast<const unsigned short *>(p));
    return fromBits(static_cast<unsigned int>(u) | (static_cast<unsigned int>(u) << 16));
  }
  __device__ __forceinline__ static PackF16 constant(float c) { return {__float2half2_rn(c)}; }
  __device__ __forceinline__ static PackF16 constantOf(const BodySrc &s) { return constant(s.value); }
  __device__ __forceinline__ static PackF16 add(PackF16 a, PackF16 b) { return {__hadd2_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackF16 sub(PackF16 a, PackF16 b) { return {__hsub2_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackF16 mul(PackF16 a, PackF16 b) { return {__hmul2_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackF16 div(PackF16 a, PackF16 b) {
    float2 fa = __half22float2(a.x), fb = __half22float2(b.x);
    return {__floats2half2_rn(__fdiv_rn(fa.x, fb.x), __fdiv_rn(fa.y, fb.y))};
  }
  __device__ __forceinline__ static PackF16 max(PackF16 a, PackF16 b) { return {__hmax2_nan(a.x, b.x)}; }
  __device__ __forceinline__ static PackF16 min(PackF16 a, PackF16 b) { return {__hmin2_nan(a.x, b.x)}; }
  __device__ __forceinline__ float lane(int i) const { return i ? __high2float(x) : __low2float(x); }
};

#endif  // AFIR_HAVE_F16

#ifdef AFIR_HAVE_BF16
struct PackBF16 {
  using Scalar = __nv_bfloat16;
  static constexpr int kLanes = 2;
  __nv_bfloat162 x;
  __device__ __forceinline__ static PackBF16 fromBits(unsigned int u) {
    PackBF16 p;
    p.x = *reinterpret_cast<__nv_bfloat162 *>(&u);
    return p;
  }
  __device__ __forceinline__ unsigned int bits() const { return *reinterpret_cast<const unsigned int *>(&x); }
  __device__ __forceinline__ static PackBF16 splat(const void *p) {
    unsigned short u = __ldg(reinterpret_cast<const unsigned short *>(p));
    return fromBits(static_cast<unsigned int>(u) | (static_cast<unsigned int>(u) << 16));
  }
  __device__ __forceinline__ static PackBF16 constant(float c) { return {__float2bfloat162_rn(c)}; }
  __device__ __forceinline__ static PackBF16 constantOf(const BodySrc &s) { return constant(s.value); }
  __device__ __forceinline__ static PackBF16 add(PackBF16 a, PackBF16 b) { return {__hadd2_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackBF16 sub(PackBF16 a, PackBF16 b) { return {__hsub2_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackBF16 mul(PackBF16 a, PackBF16 b) { return {__hmul2_rn(a.x, b.x)}; }
  __device__ __forceinline__ static PackBF16 div(PackBF16 a, PackBF16 b) {
    float2 fa = __bfloat1622float2(a.x), fb = __bfloat1622float2(b.x);
    return {__floats2bfloat162_rn(__fdiv_rn(fa.x, fb.x), __fdiv_rn(fa.y, fb.y))};
  }
  __device__ __forceinline__ static PackBF16 max(PackBF16 a, PackBF16 b) { return {__hmax2_nan(a.x, b.x)}; }
  __device__ __forceinline__ static PackBF16 min(PackBF16 a, PackBF16 b) { return {__hmin2_nan(a.x, b.x)}; }
  __device__ __forceinline__ float lane(int i) const { return i ? __high2float(x) : __low2float(x); }
};

#endif  // AFIR_HAVE_BF16

// Integer packs (afir.add/sub/mul and arith.addi/subi/muli/divsi/maxsi/minsi bodies on i32 and i16 tensors):
// two's-complement wrap-around for add, sub and mul; signed max/min; signed division truncates toward zero, a zero
// divisor gives 0 and INT_MIN / -1 gives INT_MIN (both are undefined in the IR, so any value is admissible).
struct PackI32 {
  using Scalar = int;
  static constexpr int kLanes = 1;
  int x;
  __device__ __forceinline__ static PackI32 fromBits(unsigned int u) { return {static_cast<int>(u)}; }
  __device__ __forceinline__ unsigned int bits() const { return static_cast<unsigned int>(x); }
  __device__ __forceinline__ static PackI32 splat(const void *p) { return {__ldg(reinterpret_cast<const int *>(p))}; }
  __device__ __forceinline__ static PackI32 constant(float c) { return {static_cast<int>(c)}; }
  __device__ __forceinline__ static PackI32 constantInt(int c) { return {c}; }
  __device__ __forceinline__ static PackI32 constantOf(const BodySrc &s) { return {s.ivalue}; }
  __device__ __forceinline__ static PackI32 add(PackI32 a, PackI32 b) { return fromBits(a.bits() + b.bits()); }
  __device__ __forceinline__ static PackI32 sub(PackI32 a, PackI32 b) { return fromBits(a.bits() - b.bits()); }
  __device__ __forceinline__ static PackI32 mul(PackI32 a, PackI32 b) { return fromBits(a.bits() * b.bits()); }
  __device__ __forceinline__ static int divide(int a, int b) {
    if (b == 0) return 0;
    if (b == -1) return static_cast<int>(0u - static_cast<unsigned int>(a));
    return a / b;
  }
  __device__ __forceinline__ static PackI32 div(PackI32 a, PackI32 b) { return {divide(a.x, b.x)}; }
  __device__ __forceinline__ static PackI32 max(PackI32 a, PackI32 b) { return {a.x > b.x ? a.x : b.x}; }
  __device__ __forceinline__ static PackI32 min(PackI32 a, PackI32 b) { return {a.x < b.x ? a.x : b.x}; }
  __device__ __forceinline__ float lane(int) const { return static_cast<float>(x); }
};

struct PackI16 {
  using Scalar = short;
  static constexpr int kLanes = 2;
  unsigned int x;  // two 16-bit lanes
  __device__ __forceinline__ static PackI16 fromBits(unsigned int u) { return {u}; }
  __device__ __forceinline__ unsigned int bits() const { return x; }
  __device__ __forceinline__ static PackI16 splat(const void *p) {
    const unsigned int u = __ldg(reinterpret_cast<const unsigned short *>(p));
    return {u | (u << 16)};
  }
  __device__ __forceinline__ static PackI16 constantInt(int c) {
    const unsigned int u = static_cast<unsigned int>(c) & 0xffffu;
    return {u | (u << 16)};
  }
  __device__ __forceinline__ static PackI16 constant(float c) { return constantInt(static_cast<int>(c)); }
  __device__ __forceinline__ static PackI16 constantOf(const BodySrc &s) { return constantInt(s.ivalue); }
  __device__ __forceinline__ static int lo(unsigned int v) { return static_cast<short>(v & 0xffffu); }
  __device__ __forceinline__ static int hi(unsigned int v) { return static_cast<short>(v >> 16); }
  __device__ __forceinline__ static PackI16 join(int l, int h) {
    return {(static_cast<unsigned int>(l) & 0xffffu) | (static_cast<unsigned int>(h) << 16)};
  }
  // Wrapping add / subtract of both lanes, written out: the low 15 bits of each lane in one 32-bit operation that
  // cannot carry or borrow across the lane boundary, the top bits by exclusive or.  (Not __vadd2 / __vsub2: where
  // only the low lane of the result is used -- the element-by-element loops store the low lane of a splatted value --
  // nvcc 12.9 and NVRTC 12.8 for sm_100a returned wrong low lanes for them, e.g. x + 1 for __vsub2(x, 3 in both lanes);
  // which of the two, and with a constant or a variable operand, depended on the surrounding code.)
  __device__ __forceinline__ static PackI16 add(PackI16 a, PackI16 b) {
    return {((a.x & 0x7fff7fffu) + (b.x & 0x7fff7fffu)) ^ ((a.x ^ b.x) & 0x80008000u)};
  }
  __device__ __forceinline__ static PackI16 sub(PackI16 a, PackI16 b) {
    return {((a.x | 0x80008000u) - (b.x & 0x7fff7fffu)) ^ ((a.x ^ ~b.x) & 0x80008000u)};
  }
  __device__ __forceinline__ static PackI16 mul(PackI16 a, PackI16 b) { return join(lo(a.x) * lo(b.x), hi(a.x) * hi(b.x)); }
  __device__ __forceinline__ static PackI16 div(PackI16 a, PackI16 b) {
    return join(PackI32::divide(lo(a.x), lo(b.x)), PackI32::divide(hi(a.x), hi(b.x)));
  }
  // (signed max / min lane by lane, for the same reason: no __vmaxs2 / __vmins2)
  __device__ __forceinline__ static PackI16 max(PackI16 a, PackI16 b) {
    return join(::max(lo(a.x), lo(b.x)), ::max(hi(a.x), hi(b.x)));
  }
  __device__ __forceinline__ static PackI16 min(PackI16 a, PackI16 b) {
    return join(::min(lo(a.x), lo(b.x)), ::min(hi(a.x), hi(b.x)));
  }
  __device__ __forceinline__ float lane(int i) const { return static_cast<float>(i ? hi(x) : lo(x)); }
};

// A 16-byte vector is four packs (4 x f32, 8 x f16, 8 x bf16).
template <class P> struct Vec16 {
  P p[4];
  static constexpr int kElems = 4 * P::kLanes;
  __device__ __forceinline__ static Vec16 fromRaw(const uint4 &r) {
    Vec16 v;
    v.p[0] = P::fromBits(r.x);
    v.p[1] = P::fromBits(r.y);
    v.p[2] = P::fromBits(r.z);
    v.p[3] = P::fromBits(r.w);
    return v;
  }
  __device__ __forceinline__ uint4 raw() const {
    return make_uint4(p[0].bits(), p[1].bits(), p[2].bits(), p[3].bits());
  }
  __device__ __forceinline__ static Vec16 splat(P s) {
    Vec16 v;
    v.p[0] = v.p[1] = v.p[2] = v.p[3] = s;
    return v;
  }
};

// ---- specialised bodies -------------------------------------------------------------------------
template <int ID> struct Body;
#define AFIR_BODY(ID, NVIEWS, EXPR)                                                       \
  template <> struct Body<ID> {                                                            \
    static constexpr int kViews = NVIEWS;                                                  \
    static constexpr bool kInterpreted = false;                                            \
    template <class P> __device__ __forceinline__ static P eval(const P *v, const BodyProgram &) { \
      (void)v;                                                                             \
      return EXPR;                                                                         \
    }                                                                                      \
  };
AFIR_BODY(kBodyCopy, 1, v[0])
AFIR_BODY(kBodyAdd, 2, P::add(v[0], v[1]))
AFIR_BODY(kBodyMul, 2, P::mul(v[0], v[1]))
AFIR_BODY(kBodyAddMulRhs, 2, P::mul(P::add(v[0], v[1]), v[1]))
AFIR_BODY(kBodyAddMul, 3, P::mul(P::add(v[0], v[1]), v[2]))
AFIR_BODY(kBodyMulAdd, 3, P::add(P::mul(v[0], v[1]), v[2]))
AFIR_BODY(kBodyReluAdd, 2, P::add(P::max(v[0], P::constant(0.0f)), v[1]))
AFIR_BODY(kBodyReluAddMul, 3, P::mul(P::add(P::max(v[0], P::constant(0.0f)), v[1]), v[2]))
AFIR_BODY(kBodyRelu, 1, P::max(v[0], P::constant(0.0f)))
#undef AFIR_BODY

// ---- interpreter: any chain of up to kMaxBodyOps ops over up to kMaxViews views --------------------
template <class P> __device__ __forceinline__ P interpFetch(const BodySrc &s, const P *v, const P *r, int upto) {
  if (s.kind == kSrcConst) return P::constantOf(s);
  if (s.kind == kSrcView) {
    P x = v[0];
#pragma unroll
    for (int i = 1; i < kMaxViews; ++i)
      if (s.index == i) x = v[i];
    return x;
  }
  P x = r[0];
#pragma unroll
  for (int i = 1; i < kMaxBodyOps; ++i)
    if (i < upto && s.index == i) x = r[i];
  return x;
}

template <> struct Body<kBodyInterpreted> {
  static constexpr int kViews = kMaxViews;
  static constexpr bool kInterpreted = true;
  template <class P> __device__ __forceinline__ static P eval(const P *v, const BodyProgram &prog) {
    P r[kMaxBodyOps];
#pragma unroll
    for (int i = 0; i < kMaxBodyOps; ++i) r[i] = v[0];
#pragma unroll
    for (int i = 0; i < kMaxBodyOps; ++i) {
      if (i < prog.numOps) {
        P a = interpFetch<P>(prog.ops[i].a, v, r, i);
        P b = interpFetch<P>(prog.ops[i].b, v, r, i);
        P y;
        switch (prog.ops[i].op) {
        case kOpAdd: y = P::add(a, b); break;
        case kOpSub: y = P::sub(a, b); break;
        case kOpMul: y = P::mul(a, b); break;
        case kOpDiv: y = P::div(a, b); break;
        case kOpMax: y = P::max(a, b); break;
        default: y = P::min(a, b); break;
        }
        r[i] = y;
      }
    }
    P out = v[0];
#pragma unroll
    for (int i = 0; i < kMaxBodyOps; ++i)
      if (i == prog.numOps - 1) out = r[i];
    return out;
  }
};

// ---- one 16-byte vector of every view through the body ---------------------------------------------------
// The specialised bodies simply run once per 32-bit pack.  The interpreted body would pay its op decoding and
// operand selection (select chains over every view and every earlier result) once per pack and stay far below the
// memory roofline; here it decodes an op ONCE per vector and keeps views and results as 16-byte slots in a small
// per-thread array that it indexes with the op's operand numbers (the array lives in local memory, i.e. L1:
// two 16-byte loads and one 16-byte store per op), so an op costs about a dozen instructions per vector instead
// of a few hundred.
__device__ __forceinline__ unsigned int comp(const uint4 &v, int q) { return q == 0 ? v.x : q == 1 ? v.y : q == 2 ? v.z : v.w; }

// `last` is the previous op's result: a chain op reads it from registers instead of from its slot.
template <class P>
__device__ __forceinline__ uint4 interpOperand(const BodySrc &s, const uint4 *slot, const uint4 &last, int opIndex) {
  if (s.kind == kSrcConst) {
    const unsigned int c = P::constantOf(s).bits();
    return make_uint4(c, c, c, c);
  }
  if (s.kind == kSrcOp && s.index == opIndex - 1) return last;
  return slot[s.kind == kSrcView ? s.index : kMaxViews + s.index];
}

template <class B, class P, int NV>
__device__ __forceinline__ uint4 evalVector16(const uint4 (&raw)[NV], const BodyProgram &prog) {
  if constexpr (B::kInterpreted) {
    uint4 slot[kMaxViews + kMaxBodyOps];
#pragma unroll
    for (int k = 0; k < kMaxViews; ++k)
      if (k < NV && k < prog.numViewsUsed) slot[k] = raw[k];
    uint4 last = raw[0];
    for (int i = 0; i < prog.numOps; ++i) {
      const uint4 a = interpOperand<P>(prog.ops[i].a, slot, last, i);
      const uint4 b = interpOperand<P>(prog.ops[i].b, slot, last, i);
      const P a0 = P::fromBits(a.x), a1 = P::fromBits(a.y), a2 = P::fromBits(a.z), a3 = P::fromBits(a.w);
      const P b0 = P::fromBits(b.x), b1 = P::fromBits(b.y), b2 = P::fromBits(b.z), b3 = P::fromBits(b.w);
      switch (prog.ops[i].op) {
      case kOpAdd: last = make_uint4(P::add(a0, b0).bits(), P::add(a1, b1).bits(), P::add(a2, b2).bits(), P::add(a3, b3).bits()); break;
      case kOpSub: last = make_uint4(P::sub(a0, b0).bits(), P::sub(a1, b1).bits(), P::sub(a2, b2).bits(), P::sub(a3, b3).bits()); break;
      case kOpMul: last = make_uint4(P::mul(a0, b0).bits(), P::mul(a1, b1).bits(), P::mul(a2, b2).bits(), P::mul(a3, b3).bits()); break;
      case kOpDiv: last = make_uint4(P::div(a0, b0).bits(), P::div(a1, b1).bits(), P::div(a2, b2).bits(), P::div(a3, b3).bits()); break;
      case kOpMax: last = make_uint4(P::max(a0, b0).bits(), P::max(a1, b1).bits(), P::max(a2, b2).bits(), P::max(a3, b3).bits()); break;
      default: last = make_uint4(P::min(a0, b0).bits(), P::min(a1, b1).bits(), P::min(a2, b2).bits(), P::min(a3, b3).bits()); break;
      }
      if ((prog.storeMask >> i) & 1) slot[kMaxViews + i] = last;  // only results a later, non-adjacent op reads
    }
    return last;
  } else {
    unsigned int out[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      P v[NV];
#pragma unroll
      for (int k = 0; k < NV; ++k) v[k] = P::fromBits(comp(raw[k], q));
      out[q] = B::template eval<P>(v, prog).bits();
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
  }
}

} // namespace kernels
} // namespace afir
