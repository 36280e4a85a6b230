// Broadcast + elementwise + row reduction groups: out[m] = sum_n body(views)(m, n)
// (the [parallel, reduction] linalg.generic class, lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:244-748;
// zero-initialised accumulator per :508-521; 16-bit inputs are summed as f32 and cast back,
// lib/Target/CannKernel/CannTranslation.cpp:2446-2461).
//
// HBM-bound streaming read.  L threads cooperate on one row (L = 32..CTA size), each keeping four
// 16-byte loads per view in flight; warp-shuffle tree, then a shared-memory tree across warps, f32
// accumulators throughout.  Short-and-wide problems split each row into column slices whose partial
// sums go to the workspace and are added in slice order by a second kernel (deterministic).
#include "kernels/row_reduce_skel.cuh"
#include "kernels/launch_util.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <mutex>

namespace afir {
namespace kernels {
namespace {

__device__ unsigned int g_rowReduceStatus = 0;  // wait time-outs of launches that were given no status word of their own

template <class P, int BODY, bool VECTOR, bool XCHG = false>
__global__ void __launch_bounds__(512) rowReduceKernel(const __grid_constant__ RrParams prm) {
  gridDependencyPrologue();
  rowReduceTeams<P, Body<BODY>, VECTOR, XCHG>(prm);
}

template <class P, int BODY, bool XCHG = false>
__global__ void __launch_bounds__(512, 1) rowReduceStreamKernel(const __grid_constant__ RrStreamParams prm) {
  gridDependencyPrologue();
  extern __shared__ __align__(128) unsigned char streamSmem[];
  rowReduceStream<P, Body<BODY>, XCHG>(prm, streamSmem);
}

template <class P>
__global__ void rowReduceFinalizeKernel(const float *__restrict__ partial, void *out, long long rows, int slices) {
  gridDependencyPrologue();
  rowReduceFinalize<P>(partial, out, rows, slices);
}

using KernelFn = void (*)(const RrParams);

template <class P, bool VECTOR> KernelFn pickBody(int body) {
  switch (body) {
  case kBodyCopy: return rowReduceKernel<P, kBodyCopy, VECTOR>;
  case kBodyAdd: return rowReduceKernel<P, kBodyAdd, VECTOR>;
  case kBodyMul: return rowReduceKernel<P, kBodyMul, VECTOR>;
  default: return rowReduceKernel<P, kBodyInterpreted, VECTOR>;
  }
}

// With an exchange only the add body is specialised; every other chain runs interpreted.
template <class P, bool VECTOR> KernelFn pickBodyExchange(int body) {
  return body == kBodyAdd ? rowReduceKernel<P, kBodyAdd, VECTOR, true> : rowReduceKernel<P, kBodyInterpreted, VECTOR, true>;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

} // namespace

size_t rowReduceWorkspaceBytes(int64_t rows, int splitCols) {
  return splitCols > 1 ? static_cast<size_t>(rows) * static_cast<size_t>(splitCols) * sizeof(float) : 0;
}

// Rows alone fill the machine when there are at least two CTAs' worth per SM; otherwise slice the
// columns until there are, keeping each slice at least 4096 elements long.
int chooseRowReduceSplit(int64_t rows, int64_t cols, int smCount) {
  if (rows <= 0 || cols <= 0) return 1;
  const int64_t want = 2ll * smCount;
  if (rows >= want) return 1;
  int64_t s = (want + rows - 1) / rows;
  const int64_t maxByLength = std::max<int64_t>(1, cols / 4096);
  s = std::min<int64_t>(s, maxByLength);
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(s, 1024)));
}

// Decides how a row reduction runs: 16-byte or element access, column slices, team size, and whether the
// bulk-copy staged kernel applies (and with which ring).  Pure host arithmetic: the prebuilt launch below and the
// launch of a generated kernel both follow the plan they get from here.
int planRowReduce(const RowReduceLaunch &l, int sms, RowReducePlan &plan) {
  plan = RowReducePlan();
  if (l.numViews < 1 || l.numViews > kMaxViews) return cudaErrorInvalidValue;
  const int eb = elemBytes(l.elemType);
  const int vecElems = 16 / eb;

  bool vector = l.cols % vecElems == 0;
  for (int k = 0; k < l.numViews && vector; ++k) {
    const auto &v = l.views[k];
    if (v.colStride == 1) vector = aligned16(v.base) && v.rowStride % vecElems == 0;
    else if (v.colStride != 0) vector = false;
  }
  const int perVec = vector ? vecElems : 1;
  const int64_t vecPerRow = l.cols / perVec;
  if (vecPerRow >= (1ll << 31)) return cudaErrorInvalidValue;

  int slices = l.splitCols > 0 ? l.splitCols : 1;
  if (l.exchange) {
    if (l.exchange->world < 1 || l.exchange->world > kMaxExchangeRanks || l.rows > l.exchange->slotStride) return cudaErrorInvalidValue;
    slices = 1;
  }
  slices = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(slices, std::max<int64_t>(1, vecPerRow))));
  if (slices > 1 && (!l.workspace || l.workspaceBytes < rowReduceWorkspaceBytes(l.rows, slices)))
    return cudaErrorInvalidValue;
  const int64_t vecPerSlice = (vecPerRow + slices - 1) / slices;

  // Few and very long rows (fewer than four per SM, each at least 1024 vectors): a team of 128 lanes per row leaves
  // the SMs with under 600 threads each; 256 lanes per row measured 9.6 us against 12.2 us on 512 x 16384 f32.
  const bool fewLongRows = l.ctaThreads <= 0 && l.rows < static_cast<int64_t>(sms) * 4 && vecPerSlice >= 1024;
  int threads = l.ctaThreads > 0 ? l.ctaThreads : fewLongRows ? 256 : 128;
  threads = threads >= 512 ? 512 : threads >= 256 ? 256 : threads >= 128 ? 128 : threads >= 64 ? 64 : 32;
  // team size: enough lanes that each does about one batch of four vectors, at least a warp
  int lanes = 32;
  while (lanes < threads && static_cast<int64_t>(lanes) * 4 < vecPerSlice) lanes <<= 1;
  if (l.teamLanes >= 32) {
    lanes = 32;
    while (lanes * 2 <= l.teamLanes && lanes * 2 <= threads) lanes <<= 1;
  }
  plan.vector = vector;
  plan.vecPerRow = vecPerRow;
  plan.vecPerSlice = vecPerSlice;
  plan.slices = slices;
  plan.threads = threads;
  plan.lanes = lanes;
  const int rowsPerCta = threads / lanes;
  const int64_t work = ((l.rows + rowsPerCta - 1) / rowsPerCta) * slices;
  int64_t grid = l.gridBlocks > 0 ? l.gridBlocks : work;
  plan.grid = std::max<int64_t>(1, std::min<int64_t>(grid, std::min<int64_t>(work, 0x7fffffff)));
  plan.finalizeThreads = 256;
  plan.finalizeGrid = (l.rows + plan.finalizeThreads - 1) / plan.finalizeThreads;

  // Long rows with exactly one streamed operand and enough rows to occupy every warp of the machine:
  // the bulk-copy staged kernel.
  if (vector && slices == 1 && !l.forcePlainLoads) {
    int streamed = -1, numStreamed = 0;
    for (int k = 0; k < l.numViews; ++k)
      if (l.views[k].colStride == 1) { streamed = k; ++numStreamed; }
    const int64_t rowBytes = l.cols * eb;
    int sWarps = l.ctaThreads >= 64 ? std::min(16, l.ctaThreads / 32) : kStreamWarpsDefault;
    // Not enough rows for eight warps per SM but enough for four: four-warp CTAs still take the staged loop (1024 x 8192
    // f32, the 1/8 shard of the reduction benchmark: 7.7 us against 8.9 us for the team-per-row kernel).
    if (l.ctaThreads <= 0 && l.rows < static_cast<int64_t>(sms) * sWarps && l.rows >= static_cast<int64_t>(sms) * 4) sWarps = 4;
    unsigned int sChunk = l.streamChunkBytes > 0 ? static_cast<unsigned int>(std::min(kStreamMaxChunkBytes, (l.streamChunkBytes / 512) * 512))
                                                 : static_cast<unsigned int>(kStreamChunkBytesDefault);
    if (l.streamChunkBytes <= 0 && rowBytes < static_cast<int64_t>(sChunk))  // shorter rows: one copy per row, as large as a copy can be
      sChunk = static_cast<unsigned int>(((rowBytes + 511) / 512) * 512);
    if (sChunk < 512) sChunk = 512;
    // Ring depth: what keeps HBM busy is the bytes an SM has in flight, warps x stages x chunk.  Two stages of
    // 8 KB per warp are 128 KB per SM; when short rows shrink the chunk (a copy never spans two rows) the ring
    // deepens until at least 64 KB are in flight: the producer's cursor runs ahead of the consumer's across row
    // ends, so a warp has several whole rows in flight.  64 KB and not 128: with 4 KB rows two stages (64 KB)
    // measured faster than four (65536 x 1024 f32: 41.0 against 41.9 us; 8192 x 1024: 7.27 against 8.05 us), the
    // short kernel more so because a ring of half an SM's shared memory lets the next launch's CTAs become
    // resident under this launch's tail (programmatic dependent launch).
    int sStages = l.streamStages > 0 ? std::min(32, l.streamStages) : kStreamStagesDefault;
    if (l.streamStages <= 0)
      while (sStages < 16 && static_cast<size_t>(sWarps) * sStages * sChunk < kStreamBytesInFlight) ++sStages;
    while (static_cast<size_t>(sWarps) * sStages * sChunk > 200 * 1024 && sStages > 2) --sStages;
    if (numStreamed == 1 && rowBytes >= kStreamMinRowBytes && rowBytes < (1ll << 31) &&
        l.rows >= static_cast<int64_t>(sms) * sWarps) {
      plan.staged = true;
      plan.streamedView = streamed;
      plan.streamWarps = sWarps;
      plan.streamStages = sStages;
      plan.streamChunkBytes = sChunk;
      plan.smemBytes = static_cast<size_t>(sWarps) * sStages * sChunk + static_cast<size_t>(sWarps) * sStages * sizeof(unsigned long long);
      const int64_t rowGroups = (l.rows + sWarps - 1) / sWarps;
      int64_t sgrid = l.gridBlocks > 0 ? l.gridBlocks : sms;
      sgrid = std::max<int64_t>(1, std::min<int64_t>(sgrid, rowGroups));
      if (l.exchange) sgrid = std::min<int64_t>(sgrid, sms);  // warps that wait for other ranks: one CTA per SM, all resident
      plan.grid = sgrid;
      plan.threads = sWarps * 32;
    }
  }
  return cudaSuccess;
}

namespace {
// Device address of the library's own time-out word on the current device (launches that bring no status word).
unsigned int *libraryStatusWord() {
  static std::mutex mu;
  static unsigned int *cached[64] = {nullptr};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[device]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_rowReduceStatus) == cudaSuccess) cached[device] = static_cast<unsigned int *>(p);
  }
  return cached[device];
}
} // namespace

int launchRowReduce(const RowReduceLaunch &l, cudaStream_t stream, int *launched) {
  if (launched) *launched = 0;
  if (l.rows == 0) return cudaSuccess;
  int device = 0;
  cudaGetDevice(&device);
  RowReducePlan plan;
  if (const int rc = planRowReduce(l, deviceSmCount(device), plan); rc != cudaSuccess) return rc;
  const int body = matchBody(l.body, l.numViews);

  if (plan.staged) {
    const int streamed = plan.streamedView;
    RrStreamParams sp = {};
    sp.stream = static_cast<const char *>(l.views[streamed].base);
    sp.streamRowStride = l.views[streamed].rowStride;
    for (int k = 0; k < l.numViews; ++k) {
      if (k == streamed) continue;
      sp.bcast[k] = static_cast<const char *>(l.views[k].base);
      sp.bcastRowStride[k] = l.views[k].rowStride;
    }
    sp.streamViewIndex = streamed;
    sp.numViews = l.numViews;
    sp.rows = l.rows;
    sp.rowBytes = static_cast<unsigned int>(l.cols * elemBytes(l.elemType));
    sp.stages = plan.streamStages;
    sp.chunkBytes = plan.streamChunkBytes;
    sp.out = l.out;
    sp.status = l.status ? l.status : libraryStatusWord();
    if (!sp.status) return cudaErrorInvalidValue;
    sp.prog = l.body;
    if (l.exchange) {
      sp.xchg = *l.exchange;
      // A row's entries need a store over NVLink and a poll of the local mailbox, about 4 us together, before they
      // can be read without waiting; a warp spends warps x rowBytes / (the SM's share of HBM, ~44 bytes/ns) on a row.
      const double rowNs = static_cast<double>(plan.streamWarps) * sp.rowBytes / 44.0;
      sp.finishLag = static_cast<int>(std::min(32.0, std::max(1.0, std::ceil(4000.0 / std::max(rowNs, 1.0)))));
    }
    using StreamFn = void (*)(const RrStreamParams);
    StreamFn sfn = nullptr;
    if (l.elemType == kF32) sfn = body == kBodyAdd ? rowReduceStreamKernel<PackF32, kBodyAdd> : body == kBodyCopy ? rowReduceStreamKernel<PackF32, kBodyCopy> : body == kBodyMul ? rowReduceStreamKernel<PackF32, kBodyMul> : rowReduceStreamKernel<PackF32, kBodyInterpreted>;
    else if (l.elemType == kF16) sfn = body == kBodyAdd ? rowReduceStreamKernel<PackF16, kBodyAdd> : body == kBodyCopy ? rowReduceStreamKernel<PackF16, kBodyCopy> : body == kBodyMul ? rowReduceStreamKernel<PackF16, kBodyMul> : rowReduceStreamKernel<PackF16, kBodyInterpreted>;
    else sfn = body == kBodyAdd ? rowReduceStreamKernel<PackBF16, kBodyAdd> : body == kBodyCopy ? rowReduceStreamKernel<PackBF16, kBodyCopy> : body == kBodyMul ? rowReduceStreamKernel<PackBF16, kBodyMul> : rowReduceStreamKernel<PackBF16, kBodyInterpreted>;
    if (l.exchange) {
      if (l.elemType == kF32) sfn = body == kBodyAdd ? rowReduceStreamKernel<PackF32, kBodyAdd, true> : rowReduceStreamKernel<PackF32, kBodyInterpreted, true>;
      else if (l.elemType == kF16) sfn = body == kBodyAdd ? rowReduceStreamKernel<PackF16, kBodyAdd, true> : rowReduceStreamKernel<PackF16, kBodyInterpreted, true>;
      else sfn = body == kBodyAdd ? rowReduceStreamKernel<PackBF16, kBodyAdd, true> : rowReduceStreamKernel<PackBF16, kBodyInterpreted, true>;
    }
    cudaError_t ae = cudaFuncSetAttribute(sfn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smemBytes));
    if (ae != cudaSuccess) return ae;
    launchDependent(sfn, static_cast<unsigned int>(plan.grid), plan.threads, plan.smemBytes, stream, sp);
    if (launched) *launched = 1;
    return cudaGetLastError();
  }

  RrParams p = {};
  for (int k = 0; k < l.numViews; ++k) {
    p.vbase[k] = static_cast<const char *>(l.views[k].base);
    p.rowStride[k] = l.views[k].rowStride;
    p.colStride[k] = static_cast<int>(l.views[k].colStride);
  }
  p.numViews = l.numViews;
  p.rows = l.rows;
  p.vecPerRow = static_cast<unsigned int>(plan.vecPerRow);
  p.vecPerSlice = static_cast<unsigned int>(plan.vecPerSlice);
  p.slices = plan.slices;
  p.lanesPerRow = plan.lanes;
  p.partial = static_cast<float *>(l.workspace);
  p.out = l.out;
  p.prog = l.body;
  if (l.exchange) p.xchg = *l.exchange;
  const bool vector = plan.vector;
  const int slices = plan.slices;

  KernelFn fn;
  if (l.elemType == kF32) fn = vector ? pickBody<PackF32, true>(body) : pickBody<PackF32, false>(body);
  else if (l.elemType == kF16) fn = vector ? pickBody<PackF16, true>(body) : pickBody<PackF16, false>(body);
  else fn = vector ? pickBody<PackBF16, true>(body) : pickBody<PackBF16, false>(body);
  if (l.exchange) {
    if (l.elemType == kF32) fn = vector ? pickBodyExchange<PackF32, true>(body) : pickBodyExchange<PackF32, false>(body);
    else if (l.elemType == kF16) fn = vector ? pickBodyExchange<PackF16, true>(body) : pickBodyExchange<PackF16, false>(body);
    else fn = vector ? pickBodyExchange<PackBF16, true>(body) : pickBodyExchange<PackBF16, false>(body);
  }

  launchDependent(fn, static_cast<unsigned int>(plan.grid), plan.threads, 0, stream, p);
  int n = 1;
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess && slices > 1) {
    const int ft = plan.finalizeThreads;
    const unsigned int fg = static_cast<unsigned int>(plan.finalizeGrid);
    if (l.elemType == kF32) launchDependent(rowReduceFinalizeKernel<PackF32>, fg, ft, 0, stream, p.partial, l.out, l.rows, slices);
    else if (l.elemType == kF16) launchDependent(rowReduceFinalizeKernel<PackF16>, fg, ft, 0, stream, p.partial, l.out, l.rows, slices);
    else launchDependent(rowReduceFinalizeKernel<PackBF16>, fg, ft, 0, stream, p.partial, l.out, l.rows, slices);
    n = 2;
    err = cudaGetLastError();
  }
  if (launched) *launched = n;
  return err;
}

} // namespace kernels
} // namespace afir

// ---------------------------------------------------------------------------------------------------
// Allocation-free entry point.
//
// Some hosts of this library may not allocate device memory at the moment they need a reduction:
// a real-time or inference-serving loop whose memory was sized and frozen at start-up, a process
// whose device memory is already fully committed, or a plugin running under a framework that owns
// the allocator and forbids foreign cudaMalloc calls.  The column-sliced row reduction needs scratch for its
// per-slice partial sums; the ordinary entry points take that scratch from a workspace the executor
// allocates.  This variant takes it from a fixed array inside the library image instead, so it calls
// no cudaMalloc / cudaFree and no allocating library routine.
//
// Limits and rules:
//  * rows * split_cols <= AFIRT_NO_ALLOC_MAX_PARTIALS (262 144 floats = 1 MiB; every GPU that loads
//    the library holds this array until the process exits).  Larger requests are refused.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and caches it; make that first call before starting any stream capture.
//  * The call makes `device_id` current for the launch and restores the caller's current device before it returns.
//  * All calls share the one array per device.  It keeps whatever the previous call left; nothing in
//    it has to start at zero because every slot a call reads is first written by that same call.
//    Two calls that overlap on the GPU (different streams, or different host threads) race on it:
//    serialise them.
// ---------------------------------------------------------------------------------------------------
namespace {
constexpr long long kNoAllocMaxPartials = 262144;
static __device__ __align__(256) float g_noAllocPartials[kNoAllocMaxPartials];

void noAllocFail(char *buf, size_t len, const char *msg) {
  if (!buf || len == 0) return;
  std::snprintf(buf, len, "%s", msg);
}
} // namespace

extern "C" __attribute__((visibility("default"))) int
afirt_bcast_add_rowsum_no_alloc(int device_id, int elem_type, const void *a, const void *b, void *out, int64_t rows,
                                int64_t cols, int split_cols, void *cuda_stream, char *err_buf, size_t err_len) {
  using namespace afir::kernels;
  static std::mutex mu;
  static float *scratchOnDevice[64] = {nullptr};

  if (device_id < 0 || device_id >= 64) { noAllocFail(err_buf, err_len, "device id out of range"); return 1; }
  if (elem_type != kF32 && elem_type != kF16 && elem_type != kBF16) { noAllocFail(err_buf, err_len, "elem_type must be 0 (f32), 1 (f16) or 2 (bf16)"); return 1; }
  if (rows < 0 || cols < 0 || split_cols < 1) { noAllocFail(err_buf, err_len, "rows and cols must be non-negative and split_cols at least 1"); return 1; }
  if (rows == 0) return 0;
  if (!a || !b || !out) { noAllocFail(err_buf, err_len, "a, b and out are required"); return 1; }
  // rows > max / split_cols instead of rows * split_cols > max: the product of two caller-chosen numbers can wrap
  if (split_cols > kNoAllocMaxPartials || rows > kNoAllocMaxPartials / split_cols) {
    char msg[200];
    std::snprintf(msg, sizeof(msg), "rows (%lld) x split_cols (%d) exceeds the built-in scratch of %lld partial sums",
                  static_cast<long long>(rows), split_cols, kNoAllocMaxPartials);
    noAllocFail(err_buf, err_len, msg);
    return 1;
  }
  // rows is at most 262 144 from here on; keep rows * cols * element size inside 63 bits before pointers are formed
  if (cols > (1ll << 40)) { noAllocFail(err_buf, err_len, "cols exceeds 2^40"); return 1; }
  // The launch needs `device_id` current; the caller's current device is put back before returning, on every path.
  struct DeviceScope {
    int previous = -1;
    ~DeviceScope() { if (previous >= 0) cudaSetDevice(previous); }
  } scope;
  int current = -1;
  cudaError_t e = cudaGetDevice(&current);
  if (e != cudaSuccess) { noAllocFail(err_buf, err_len, cudaGetErrorString(e)); return 1; }
  if (current != device_id) {
    e = cudaSetDevice(device_id);
    if (e != cudaSuccess) { noAllocFail(err_buf, err_len, cudaGetErrorString(e)); return 1; }
    scope.previous = current;
  }
  float *scratch = nullptr;
  {
    // The array's name is only a host-side handle; the kernel needs its address in this device's memory.
    std::lock_guard<std::mutex> lock(mu);
    if (!scratchOnDevice[device_id]) {
      void *p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noAllocPartials);
      if (e != cudaSuccess || !p) {
        noAllocFail(err_buf, err_len, e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned null");
        return 1;
      }
      scratchOnDevice[device_id] = static_cast<float *>(p);
    }
    scratch = scratchOnDevice[device_id];
  }

  RowReduceLaunch l = {};
  l.elemType = elem_type;
  l.rows = rows;
  l.cols = cols;
  l.numViews = 2;
  l.views[0].base = a;  // a[m]: follows the row, broadcast along the columns
  l.views[0].rowStride = 1;
  l.views[0].colStride = 0;
  l.views[1].base = b;  // b[m, n]
  l.views[1].rowStride = cols;
  l.views[1].colStride = 1;
  l.out = out;
  l.body.numOps = 1;
  l.body.ops[0].op = kOpAdd;
  l.body.ops[0].a = {kSrcView, 0, 0.0f};
  l.body.ops[0].b = {kSrcView, 1, 0.0f};
  l.splitCols = split_cols;
  l.workspace = scratch;
  l.workspaceBytes = static_cast<size_t>(kNoAllocMaxPartials) * sizeof(float);
  int launched = 0;
  const int rc = launchRowReduce(l, static_cast<cudaStream_t>(cuda_stream), &launched);
  if (rc != 0) { noAllocFail(err_buf, err_len, cudaGetErrorString(static_cast<cudaError_t>(rc))); return 1; }
  return 0;
}

namespace afir {
namespace kernels {
int rowReduceCheckStatus(int device, char *errorText) {
  (void)device;
  unsigned int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_rowReduceStatus, sizeof(status)) != cudaSuccess) return 0;
  if (status == 0) return 0;
  const unsigned int zero = 0;
  cudaMemcpyToSymbol(g_rowReduceStatus, &zero, sizeof(zero));
  if (errorText) std::snprintf(errorText, 256, "row reduction: a warp gave up waiting for a bulk copy after 2 s");
  return 1;
}
} // namespace kernels
} // namespace afir
