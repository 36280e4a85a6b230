#include "kernels/row_reduce_skel.cuh"
// Generated for one fused group; the loops are the function templates of kernels/*_skel.cuh.
using namespace afir::kernels;

// Tells the runtime that every kernel of this module begins with gridDependencyPrologue().
extern "C" __global__ void afir_waits_for_grid_dependencies() {}

// all-int64 TilingData: the descriptor's fields in order, then the words the runtime fills in at launch
struct TilingData {
  long long CTA_THREADS;
  long long TEAM_LANES;
  long long SPLIT_N;
  long long BULK_COPY;
  long long STREAM_STAGES;
  long long STREAM_CHUNK;
  long long dim_arg0_0;
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

extern "C" __global__ void __launch_bounds__(512) broadcast_add_reduce(const void *arg0, const void *arg1, void *arg2, void *workspace, const __grid_constant__ TilingData t) {
  gridDependencyPrologue();
  if (t.afir_row_end >= 0 && t.afir_row_end <= t.afir_row_begin) return;  // empty row window
  const long long rowb = t.afir_row_end >= 0 ? t.afir_row_begin : 0;
  (void)workspace; (void)rowb;
  {
    const long long rows0 = t.afir_row_end >= 0 ? t.afir_row_end - t.afir_row_begin : t.dim_arg1_0;
    RrParams prm = {};
    prm.vbase[0] = static_cast<const char *>(arg0) + (rowb * (1LL)) * 4; prm.rowStride[0] = 1LL; prm.colStride[0] = 0;
    prm.vbase[1] = static_cast<const char *>(arg1) + (rowb * (t.dim_arg1_1)) * 4; prm.rowStride[1] = t.dim_arg1_1; prm.colStride[1] = 1;
    prm.numViews = 2;
    prm.rows = rows0;
    const bool vec = t.afir_p0 != 0;
    prm.vecPerRow = static_cast<unsigned int>((t.dim_arg1_1) / (vec ? 4 : 1));
    prm.slices = static_cast<int>(t.afir_p1);
    prm.vecPerSlice = static_cast<unsigned int>(t.afir_p2);
    prm.lanesPerRow = static_cast<int>(t.afir_p3);
    prm.partial = reinterpret_cast<float *>(static_cast<char *>(workspace) + 256);
    prm.out = static_cast<char *>(arg2) + (rowb * (1LL)) * 4;
    if (vec) rowReduceTeams<PackF32, FusedBody0, true>(prm);
    else rowReduceTeams<PackF32, FusedBody0, false>(prm);
  }
}

extern "C" __global__ void __launch_bounds__(512, 1) broadcast_add_reduce__staged(const void *arg0, const void *arg1, void *arg2, void *workspace, const __grid_constant__ TilingData t) {
  extern __shared__ __align__(128) unsigned char streamSmem[];
  gridDependencyPrologue();
  if (t.afir_row_end >= 0 && t.afir_row_end <= t.afir_row_begin) return;  // empty row window
  const long long rowb = t.afir_row_end >= 0 ? t.afir_row_begin : 0;
  (void)workspace; (void)rowb;
  {
    const long long rows0 = t.afir_row_end >= 0 ? t.afir_row_end - t.afir_row_begin : t.dim_arg1_0;
    RrStreamParams sp = {};
    sp.bcast[0] = static_cast<const char *>(arg0) + (rowb * (1LL)) * 4; sp.bcastRowStride[0] = 1LL;
    sp.stream = static_cast<const char *>(arg1) + (rowb * (t.dim_arg1_1)) * 4; sp.streamRowStride = t.dim_arg1_1;
    sp.streamViewIndex = 1;
    sp.numViews = 2;
    sp.rows = rows0;
    sp.rowBytes = static_cast<unsigned int>((t.dim_arg1_1) * 4);
    sp.stages = static_cast<int>(t.afir_p0);
    sp.chunkBytes = static_cast<unsigned int>(t.afir_p1);
    sp.out = static_cast<char *>(arg2) + (rowb * (1LL)) * 4;
    sp.status = reinterpret_cast<unsigned int *>(static_cast<char *>(workspace) + 8);
    rowReduceStream<PackF32, FusedBody0>(sp, streamSmem);
  }
}

extern "C" __global__ void  broadcast_add_reduce__finalize(const void *arg0, const void *arg1, void *arg2, void *workspace, const __grid_constant__ TilingData t) {
  gridDependencyPrologue();
  if (t.afir_row_end >= 0 && t.afir_row_end <= t.afir_row_begin) return;  // empty row window
  const long long rowb = t.afir_row_end >= 0 ? t.afir_row_begin : 0;
  (void)workspace; (void)rowb;
  {
    const long long rows0 = t.afir_row_end >= 0 ? t.afir_row_end - t.afir_row_begin : t.dim_arg1_0;
    rowReduceFinalize<PackF32>(reinterpret_cast<const float *>(static_cast<char *>(workspace) + 256), static_cast<char *>(arg2) + (rowb * (1LL)) * 4, rows0, static_cast<int>(t.afir_p1));
  }
}
