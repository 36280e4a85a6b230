// Shared device-side pieces of the bandwidth-bound fused-group kernels: 16-byte vector packs per
// element type, per-op-rounded arithmetic, the specialised body functors and the body interpreter.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels/kernels.h"

namespace afir {
namespace kernels {

// ---- 32-bit division by a launch-time constant ------------------------------------------------
struct FastDiv {
  unsigned int magic;
  unsigned int shift;
  unsigned int divisor;
};
inline FastDiv makeFastDiv(unsigned int d) {
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
  __device__ __forceinline__ static PackI16 constant(float c) {
    const unsigned int u = static_cast<unsigned int>(static_cast<int>(c)) & 0xffffu;
    return {u | (u << 16)};
  }
  __device__ __forceinline__ static int lo(unsigned int v) { return static_cast<short>(v & 0xffffu); }
  __device__ __forceinline__ static int hi(unsigned int v) { return static_cast<short>(v >> 16); }
  __device__ __forceinline__ static PackI16 join(int l, int h) {
    return {(static_cast<unsigned int>(l) & 0xffffu) | (static_cast<unsigned int>(h) << 16)};
  }
  __device__ __forceinline__ static PackI16 add(PackI16 a, PackI16 b) { return {__vadd2(a.x, b.x)}; }
  __device__ __forceinline__ static PackI16 sub(PackI16 a, PackI16 b) { return {__vsub2(a.x, b.x)}; }
  __device__ __forceinline__ static PackI16 mul(PackI16 a, PackI16 b) { return join(lo(a.x) * lo(b.x), hi(a.x) * hi(b.x)); }
  __device__ __forceinline__ static PackI16 div(PackI16 a, PackI16 b) {
    return join(PackI32::divide(lo(a.x), lo(b.x)), PackI32::divide(hi(a.x), hi(b.x)));
  }
  __device__ __forceinline__ static PackI16 max(PackI16 a, PackI16 b) { return {__vmaxs2(a.x, b.x)}; }
  __device__ __forceinline__ static PackI16 min(PackI16 a, PackI16 b) { return {__vmins2(a.x, b.x)}; }
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
  if (s.kind == kSrcConst) return P::constant(s.value);
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

} // namespace kernels
} // namespace afir
