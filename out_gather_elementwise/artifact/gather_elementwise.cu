#include "kernels/gather_skel.cuh"
// Generated for one fused group; the loops are the function templates of kernels/*_skel.cuh.
using namespace afir::kernels;

// all-int64 TilingData: the descriptor's fields in order, then the words the runtime fills in at launch
struct TilingData {
  long long CTA_THREADS;
  long long UNROLL;
  long long BULK_COPY;
  long long STREAM_STAGES;
  long long STREAM_ROWS;
  long long STREAM_WARPS;
  long long dim_arg0_0;
  long long dim_arg0_1;
  long long dim_arg1_0;
  long long dim_arg2_0;
  long long dim_arg3_0;
  long long dim_arg3_1;
  long long afir_row_begin, afir_row_end;  // window of the leading iteration dim; afir_row_end < 0 = all of it
  long long afir_p0, afir_p1, afir_p2, afir_p3, afir_p4, afir_p5;  // launch plan
};

struct FusedBody0 {
  static constexpr int kViews = 3;
  static constexpr bool kInterpreted = false;
  template <class P> __device__ __forceinline__ static P eval(const P *v, const afir::kernels::BodyProgram &) {
    const P r0 = P::mul(v[0], v[1]);
    const P r1 = P::add(r0, v[2]);
    return r1;
  }
};

template <bool PAIR>
__device__ __forceinline__ void gather_elementwise__body(const void *arg0, const void *arg1, const void *arg2, const void *arg3, void *arg4, void *workspace, const TilingData &t) {
  if (t.afir_row_end >= 0 && t.afir_row_end <= t.afir_row_begin) return;  // empty row window
  const long long rowb = t.afir_row_end >= 0 ? t.afir_row_begin : 0;
  (void)workspace; (void)rowb;
  {
    const long long rows0 = t.afir_row_end >= 0 ? t.afir_row_end - t.afir_row_begin : t.dim_arg1_0;
    GaParams prm = {};
    prm.table = static_cast<const char *>(arg0);
    prm.tableRows = t.dim_arg0_0; prm.tableCols = t.dim_arg0_1; prm.tableRowStride = t.dim_arg0_1;
    prm.indices = static_cast<const char *>(arg1) + rowb * 4;
    prm.index64 = 0;
    prm.vbase[1] = static_cast<const char *>(arg2); prm.rowStride[1] = 0LL; prm.colStride[1] = 1;
    prm.vbase[2] = static_cast<const char *>(arg3) + (rowb * (t.dim_arg3_1)) * 2; prm.rowStride[2] = t.dim_arg3_1; prm.colStride[2] = 1;
    prm.numViews = 3;
    prm.out = static_cast<char *>(arg4) + (rowb * (t.dim_arg0_1)) * 2;
    prm.outRowStride = t.dim_arg0_1;
    prm.status = static_cast<unsigned long long *>(workspace);
    const long long cols = t.dim_arg0_1;
    const bool vec = cols % 8 == 0 && ((reinterpret_cast<unsigned long long>(prm.table) & 15ull) == 0ull) && prm.tableRowStride % 8 == 0 && ((reinterpret_cast<unsigned long long>(prm.vbase[1]) & 15ull) == 0ull) && prm.rowStride[1] % 8 == 0 && ((reinterpret_cast<unsigned long long>(prm.vbase[2]) & 15ull) == 0ull) && prm.rowStride[2] % 8 == 0 && ((reinterpret_cast<unsigned long long>(prm.out) & 15ull) == 0ull) && prm.outRowStride % 8 == 0;
    prm.vecPerRow = static_cast<unsigned int>(vec ? cols / 8 : cols);
    // multiply-shift constants of the division by vecPerRow, prepared by the host for both access widths
    const unsigned long long mg = static_cast<unsigned long long>(vec ? t.afir_p1 : t.afir_p2);
    prm.divVpr.magic = static_cast<unsigned int>(mg); prm.divVpr.shift = static_cast<unsigned int>(mg >> 32); prm.divVpr.divisor = prm.vecPerRow;
    prm.totalVec = static_cast<unsigned int>(rows0 * prm.vecPerRow);
    const unsigned int inFlight = t.afir_p0 == 1 ? 1u : 2u;
    if (!vec) gatherRowsTiles<PackBF16, FusedBody0, 2, false>(prm);
    else if (!PAIR || inFlight == 1u) gatherRowsTiles<PackBF16, FusedBody0, 1, true>(prm);
    else gatherRowsTiles<PackBF16, FusedBody0, 2, true>(prm);
  }
}

extern "C" __global__ void __launch_bounds__(512) gather_elementwise(const void *arg0, const void *arg1, const void *arg2, const void *arg3, void *arg4, void *workspace, const __grid_constant__ TilingData t) {
  gather_elementwise__body<true>(arg0, arg1, arg2, arg3, arg4, workspace, t);
}

// one vector per thread in flight (the default plan): the entry the runtime launches unless the plan asks for two
extern "C" __global__ void __launch_bounds__(512) gather_elementwise__one(const void *arg0, const void *arg1, const void *arg2, const void *arg3, void *arg4, void *workspace, const __grid_constant__ TilingData t) {
  gather_elementwise__body<false>(arg0, arg1, arg2, arg3, arg4, workspace, t);
}
