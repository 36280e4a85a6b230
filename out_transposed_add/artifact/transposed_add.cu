#include "kernels/elementwise_blocks_skel.cuh"
// Generated for one fused group; the loops are the function templates of kernels/*_skel.cuh.
using namespace afir::kernels;

// Tells the runtime that every kernel of this module begins with gridDependencyPrologue().
extern "C" __global__ void afir_waits_for_grid_dependencies() {}

// Tells the runtime that this module's kernel is launched with CTAs of 256 threads.
extern "C" __global__ void afir_ctas_of_256_threads() {}

// all-int64 TilingData: the descriptor's fields in order, then the words the runtime fills in at launch
struct TilingData {
  long long CTA_THREADS;
  long long UNROLL;
  long long dim_arg0_0;
  long long dim_arg0_1;
  long long dim_arg1_0;
  long long dim_arg1_1;
  long long afir_row_begin, afir_row_end;  // window of the leading iteration dim; afir_row_end < 0 = all of it
  long long afir_p0, afir_p1, afir_p2, afir_p3, afir_p4, afir_p5;  // launch plan
};

struct FusedBody0 {
  static constexpr int kViews = 2;
  static constexpr bool kInterpreted = false;
  template <class P> __device__ __forceinline__ static P eval(const P *v, const afir::kernels::BodyProgram &) {
    const P r0 = P::add(v[0], v[1]);
    return r0;
  }
};

extern "C" __global__ void __launch_bounds__(256, 3) transposed_add(const void *arg0, const void *arg1, void *arg2, void *workspace, const __grid_constant__ TilingData t) {
  gridDependencyPrologue();
  if (t.afir_row_end >= 0 && t.afir_row_end <= t.afir_row_begin) return;  // empty row window
  const long long rowb = t.afir_row_end >= 0 ? t.afir_row_begin : 0;
  (void)workspace; (void)rowb;
  {  // group 0
    const long long rows0 = t.afir_row_end >= 0 ? t.afir_row_end - t.afir_row_begin : t.dim_arg1_0;
    EwParams prm = {};
    const long long d0 = 1LL, d1 = rows0, d2 = t.dim_arg1_1;
    prm.vbase[0] = static_cast<const char *>(arg0) + (rowb * (1LL)) * 2;
    prm.vs0[0] = 0LL; prm.vs1[0] = 1LL; prm.vs2[0] = t.dim_arg0_1;
    prm.vbase[1] = static_cast<const char *>(arg1) + (rowb * (t.dim_arg1_1)) * 2;
    prm.vs0[1] = 0LL; prm.vs1[1] = t.dim_arg1_1; prm.vs2[1] = 1LL;
    prm.obase = static_cast<char *>(arg2) + (rowb * (t.dim_arg1_1)) * 2;
    prm.os0 = 0LL; prm.os1 = t.dim_arg1_1;
    const bool vec = false;
    const long long vpr = vec ? d2 / 8 : d2;
    prm.vecPerRow = static_cast<unsigned int>(vpr);
    prm.d1 = static_cast<unsigned int>(d1);
    prm.totalVec = static_cast<unsigned int>(d0 * d1 * vpr);
    prm.flat = (d0 == 1 && d1 == 1) ? 1 : 0;
    prm.numViews = 2;
    const unsigned int tileVecs = blockDim.x * 2u;
    prm.numTiles = (prm.totalVec + tileVecs - 1u) / tileVecs;
    EbParams bp = {};
    bp.vbase[0] = prm.vbase[0]; bp.s0[0] = prm.vs0[0]; bp.s1[0] = prm.vs1[0]; bp.s2[0] = prm.vs2[0]; bp.kind[0] = kViewTransposed;
    bp.vbase[1] = prm.vbase[1]; bp.s0[1] = prm.vs0[1]; bp.s1[1] = prm.vs1[1]; bp.s2[1] = prm.vs2[1]; bp.kind[1] = kViewRowMajor;
    bp.numViews = 2; bp.obase = prm.obase; bp.os0 = prm.os0; bp.os1 = prm.os1; bp.d1 = d1; bp.d2 = d2;
    bp.tilesX = static_cast<unsigned int>((d2 + 255) / 256);
    bp.tilesY = static_cast<unsigned int>((d1 + 63) / 64);
    bp.numTiles = static_cast<unsigned long long>(d0) * bp.tilesX * bp.tilesY;
    if (blockDim.x == 256u && ((reinterpret_cast<unsigned long long>(prm.obase) & 15ull) == 0ull) && prm.os0 % 8 == 0 && prm.os1 % 8 == 0 && ((reinterpret_cast<unsigned long long>(prm.vbase[0]) & 15ull) == 0ull) && prm.vs0[0] % 8 == 0 && prm.vs2[0] % 8 == 0 && ((reinterpret_cast<unsigned long long>(prm.vbase[1]) & 15ull) == 0ull) && prm.vs0[1] % 8 == 0 && prm.vs1[1] % 8 == 0) elementwiseBlocksTiles<PackF16, FusedBody0, 2>(bp);
    else elementwiseTiles<PackF16, FusedBody0, 2, false, false, true>(prm);
  }
}
