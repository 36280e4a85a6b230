// E x E element blocks held in registers as E 16-byte rows (E = 16 / element bytes) and their transpose:
// byte permutes for 16-bit elements, pure register renaming for 32-bit ones.  Used by the transpose kernel
// and by the elementwise kernel for operands that are read through a transposed view.
#pragma once

#ifndef __CUDACC_RTC__
#include <cuda_runtime.h>
#endif

namespace afir {
namespace kernels {

template <int EB> struct RegBlock;

template <> struct RegBlock<4> {  // 4 x 4 words: out[c].word[r] = in[r].word[c]
  static constexpr int kEdge = 4;
  __device__ __forceinline__ static void transpose(const uint4 (&a)[4], uint4 (&o)[4]) {
    o[0] = make_uint4(a[0].x, a[1].x, a[2].x, a[3].x);
    o[1] = make_uint4(a[0].y, a[1].y, a[2].y, a[3].y);
    o[2] = make_uint4(a[0].z, a[1].z, a[2].z, a[3].z);
    o[3] = make_uint4(a[0].w, a[1].w, a[2].w, a[3].w);
  }
};

template <> struct RegBlock<2> {  // 8 x 8 halfwords
  static constexpr int kEdge = 8;
  __device__ __forceinline__ static unsigned int word(const uint4 &v, int w) { return w == 0 ? v.x : w == 1 ? v.y : w == 2 ? v.z : v.w; }
  __device__ __forceinline__ static void transpose(const uint4 (&a)[8], uint4 (&o)[8]) {
    // Rows 2A and 2A+1 hold the 2 x 2 block (A, W) in word W.  Output row 2W+p, word A is that block's column p:
    // the low (p = 0) or high (p = 1) halfwords of the two rows, lower row first.
#pragma unroll
    for (int W = 0; W < 4; ++W) {
      unsigned int lo[4], hi[4];
#pragma unroll
      for (int A = 0; A < 4; ++A) {
        const unsigned int r0 = word(a[2 * A], W), r1 = word(a[2 * A + 1], W);
        lo[A] = __byte_perm(r0, r1, 0x5410);
        hi[A] = __byte_perm(r0, r1, 0x7632);
      }
      o[2 * W] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      o[2 * W + 1] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    }
  }
};

} // namespace kernels
} // namespace afir
