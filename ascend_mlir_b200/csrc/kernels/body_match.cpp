// Host-side analysis of fused bodies: which straight-line specialisation (if any) computes a given op chain, and
// the bookkeeping the interpreter wants.  No CUDA in this file: the descriptor parser and the compiler front-end
// tools link it without the kernel objects.
#include <algorithm>

#include "kernels/kernels.h"

namespace afir {
namespace kernels {

namespace {
bool srcIs(const BodySrc &s, int kind, int index) { return s.kind == kind && s.index == index; }
bool srcIsZero(const BodySrc &s) { return s.kind == kSrcConst && s.value == 0.0f; }
// op(a,b) with commutative matching for add/mul/max/min
bool opIs(const BodyOp &o, int code, int ak, int ai, int bk, int bi) {
  if (o.op != code) return false;
  if (srcIs(o.a, ak, ai) && srcIs(o.b, bk, bi)) return true;
  bool commutative = code == kOpAdd || code == kOpMul || code == kOpMax || code == kOpMin;
  return commutative && srcIs(o.a, bk, bi) && srcIs(o.b, ak, ai);
}
bool isRelu(const BodyOp &o, int view) {
  return o.op == kOpMax && ((srcIs(o.a, kSrcView, view) && srcIsZero(o.b)) || (srcIs(o.b, kSrcView, view) && srcIsZero(o.a)));
}
} // namespace

void finishBodyProgram(BodyProgram &prog) {
  int views = 1;
  unsigned int mask = 0;
  for (int i = 0; i < prog.numOps && i < kMaxBodyOps; ++i) {
    for (const BodySrc *s : {&prog.ops[i].a, &prog.ops[i].b}) {
      if (s->kind == kSrcView) views = std::max(views, s->index + 1);
      if (s->kind == kSrcOp && s->index != i - 1 && s->index >= 0 && s->index < kMaxBodyOps) mask |= 1u << s->index;
    }
  }
  prog.numViewsUsed = std::min(views, kMaxViews);
  prog.storeMask = mask;
}

int matchBody(const BodyProgram &p, int numViews) {
  const BodyOp *o = p.ops;
  if (p.numOps == 0 && numViews >= 1) return kBodyCopy;
  if (p.numOps == 1) {
    if (opIs(o[0], kOpAdd, kSrcView, 0, kSrcView, 1)) return kBodyAdd;
    if (opIs(o[0], kOpMul, kSrcView, 0, kSrcView, 1)) return kBodyMul;
    if (isRelu(o[0], 0)) return kBodyRelu;
  }
  if (p.numOps == 2) {
    if (opIs(o[0], kOpAdd, kSrcView, 0, kSrcView, 1) && opIs(o[1], kOpMul, kSrcOp, 0, kSrcView, 1)) return kBodyAddMulRhs;
    if (opIs(o[0], kOpAdd, kSrcView, 0, kSrcView, 1) && opIs(o[1], kOpMul, kSrcOp, 0, kSrcView, 2)) return kBodyAddMul;
    if (opIs(o[0], kOpMul, kSrcView, 0, kSrcView, 1) && opIs(o[1], kOpAdd, kSrcOp, 0, kSrcView, 2)) return kBodyMulAdd;
    if (isRelu(o[0], 0) && opIs(o[1], kOpAdd, kSrcOp, 0, kSrcView, 1)) return kBodyReluAdd;
  }
  if (p.numOps == 3) {
    if (isRelu(o[0], 0) && opIs(o[1], kOpAdd, kSrcOp, 0, kSrcView, 1) && opIs(o[2], kOpMul, kSrcOp, 1, kSrcView, 2))
      return kBodyReluAddMul;
  }
  return kBodyInterpreted;
}

} // namespace kernels
} // namespace afir
