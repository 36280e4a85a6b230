// Gather + elementwise fused groups.
//   axis 0, row gather:    out[i, j] = body(table[idx[i], j], views...)   -- the "embedding" form the
//       reference's structured-op marker tags as embedding_dim
//       (lib/Conversion/MarkStructuredOps/MarkStructuredOpsPass.cpp:54-139) and leaves unlowered
//       (lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:833-839);
//   axis 1, column gather: out[i, j] = body(table[i, idx[j]], views...)   -- the index_select form it
//       lowers (ComputeConversion.cpp:847-1273), pre-op -> extract -> post-op order per
//       lib/Conversion/FuseGatherElementwise/FuseGatherElementwisePass.cpp:190-274.
// A pre-op on the table commutes with the gather, so it is simply the first op of the body.
//
// HBM-bound.  Row gather: consecutive threads take consecutive 16-byte pieces of one gathered row,
// so a 512-byte row is one fully coalesced warp request; each thread keeps UNROLL rows in flight
// (indices first, then table pieces + the other views).  Column gather: each thread produces one
// 16-byte output vector from scalar loads of the (cache-resident) table row.
// Indices outside the table raise *status and leave the output untouched; nothing is clamped.
#include "kernels/gather_skel.cuh"
#include "kernels/launch_util.h"

#include <algorithm>

namespace afir {
namespace kernels {
namespace {

template <class P, int BODY, int UNROLL, bool VECTOR, bool SHARDED = false>
__global__ void __launch_bounds__(512) gatherRowsKernel(const __grid_constant__ GaParams prm) {
  gatherRowsTiles<P, Body<BODY>, UNROLL, VECTOR, SHARDED>(prm);
}

// ---- axis 1 ------------------------------------------------------------------------------------
// One output element per thread-iteration (the table accesses are scattered anyway; consecutive
// threads still write consecutive output elements).
template <class P, int BODY>
__global__ void __launch_bounds__(512) gatherColsKernel(const __grid_constant__ GaParams prm) {
  using B = Body<BODY>;
  constexpr int NV = B::kViews;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
  const unsigned int stride = gridDim.x * blockDim.x;
  for (unsigned int g = blockIdx.x * blockDim.x + threadIdx.x; g < prm.totalVec; g += stride) {
    const unsigned int row = fastDivide(g, prm.divVpr);
    const unsigned int col = g - row * prm.vecPerRow;
    const long long src = loadIndex(prm.indices, col, prm.index64);
    if (src < 0 || src >= prm.tableCols) {
      if (row == 0 && prm.status) atomicAdd(prm.status, 1ull);
      continue;
    }
    P v[NV];
    v[0] = P::splat(prm.table + (static_cast<long long>(row) * prm.tableRowStride + src) * kElemBytes);
#pragma unroll
    for (int k = 1; k < NV; ++k) {
      v[k] = v[0];
      if (k < prm.numViews)
        v[k] = P::splat(prm.vbase[k] + (static_cast<long long>(row) * prm.rowStride[k] +
                                        static_cast<long long>(col) * prm.colStride[k]) * kElemBytes);
    }
    storeOne<P>(prm.out + (static_cast<long long>(row) * prm.outRowStride + col) * kElemBytes,
                B::template eval<P>(v, prm.prog));
  }
}

// ---- axis 0, bulk-copy staged variant (opt-in) ----------------------------------------------------------
// Measured result first: on B200 this variant is SLOWER than the plain kernel above for every row length tried
// (bf16, 403 MB of algorithmic traffic: rows of 256 B 70 vs 65 us, 512 B 71 vs 65 us, 2 KB 76 vs 64 us, 8 KB 123
// vs 64 us), whatever the ring depth, rows per stage or warp count: the copy engine completes about one 512-byte
// row copy per 80 cycles per SM, which caps scattered-row traffic below what 2048 resident threads with one
// 16-byte load each sustain.  It stays as a tiling candidate (BULK_COPY = 1) and as the record of that experiment.
//
// The plain kernel keeps 32 bytes per thread in flight (one table piece and one piece of a streamed
// view) and its table loads wait for an index load first, so at full occupancy an SM has about 64 KB in
// flight, which is what HBM latency x bandwidth needs and no more.  Here every warp owns a ring of stages in
// shared memory; a stage holds G gathered table rows and the same G rows of every streamed view, all brought
// in by cp.async.bulk (one copy per gathered row, issued by the lane that read its index; one copy per view
// when its rows are contiguous).  The warp computes the body from shared memory and stores the results from
// registers with coalesced 16-byte stores, then refills the stage.  Indices are read one stage ahead.  Bytes in flight no longer depend on
// registers or occupancy: 8 warps x 2 stages in flight x 8 KB = 128 KB per SM by default.
// Out-of-range indices are counted in *status; their rows are neither read nor written.  Every wait on a
// stage barrier is bounded (2 s); on timeout the warp sets bit 62 of *status, gives its other stages one more bounded wait and returns.
constexpr unsigned long long kGatherTimeoutFlag = 1ull << 62;
constexpr unsigned long long kGatherWaitLimitNs = 2000000000ull;
constexpr int kMaxStreamedViews = 2;

struct GaStreamParams {
  const char *table;
  long long tableRows;
  long long tableRowStrideBytes;
  const void *indices;
  int index64;
  // views other than the table: streamed (one row per output row) or broadcast along rows (same row for all)
  const char *vbase[kMaxViews];
  long long rowStrideBytes[kMaxViews];  // 0 = broadcast along rows
  int slot[kMaxViews];                  // streamed views: which stage buffer (1..), else -1
  int numViews;
  int numStreamed;
  char *out;
  long long outRowStrideBytes;
  long long rows;
  unsigned int rowBytes;      // multiple of 16
  unsigned int vecPerRow;     // rowBytes / 16
  FastDiv divVpr;
  int rowsPerStage;           // G <= 32
  int stages;
  unsigned long long *status;
  BodyProgram prog;
};

__device__ __forceinline__ unsigned int gaSmemU32(const void *p) { return static_cast<unsigned int>(__cvta_generic_to_shared(p)); }

// Waits until the barrier's phase with this parity has completed, or gives up after kGatherWaitLimitNs.
__device__ __forceinline__ bool gaWaitStage(unsigned int bar, unsigned int parity) {
  unsigned int done = 0, spins = 0;
  unsigned long long t0 = 0;
  while (true) {
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((++spins & 255u) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > kGatherWaitLimitNs) return false;
    }
  }
}

template <class P, int BODY>
__global__ void __launch_bounds__(512, 1) gatherRowsStreamKernel(const __grid_constant__ GaStreamParams prm) {
  using B = Body<BODY>;
  constexpr int NV = B::kViews;
  extern __shared__ __align__(128) unsigned char gaSmem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int G = prm.rowsPerStage, S = prm.stages;
  const unsigned int bufBytes = static_cast<unsigned int>(G) * prm.rowBytes;      // one view's rows of a stage
  const unsigned int stageBytes = bufBytes * static_cast<unsigned int>(1 + prm.numStreamed);
  unsigned char *ring = gaSmem + static_cast<size_t>(warp) * S * stageBytes;
  const unsigned int ringU32 = gaSmemU32(ring);
  unsigned long long *bars = reinterpret_cast<unsigned long long *>(gaSmem + static_cast<size_t>(warps) * S * stageBytes) + warp * S;

  if (lane == 0) {
    for (int s = 0; s < S; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gaSmemU32(&bars[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  // Every warp owns one contiguous range of rows (a multiple of 32 long), walked in chunks of G rows.  Indices
  // are read 32 at a time, one coalesced load per block of 32 rows, two blocks ahead of the copies that use
  // them, so no copy ever waits for an index load; lane g < G of a chunk gets its index by shuffle.
  const long long totalWarps = static_cast<long long>(gridDim.x) * warps;
  const long long rowsPerWarp = ((prm.rows + totalWarps - 1) / totalWarps + 31) / 32 * 32;
  const long long rangeBegin = min(prm.rows, (static_cast<long long>(blockIdx.x) * warps + warp) * rowsPerWarp);
  const long long rangeEnd = min(prm.rows, rangeBegin + rowsPerWarp);
  const long long firstChunk = rangeBegin / G;                // G divides 32, so ranges start on chunk boundaries
  const long long numChunks = rangeBegin < rangeEnd ? (rangeEnd + G - 1) / G : firstChunk;  // one past this warp's last chunk
  const int chunksPerBlock = 32 / G;
  auto readIndexBlock = [&](long long block) -> long long {   // block = index of a group of 32 rows of the range
    const long long row = rangeBegin + block * 32 + lane;
    return row < rangeEnd ? loadIndex(prm.indices, row, prm.index64) : -1;
  };
  long long idxBlockNow = readIndexBlock(0), idxBlockNext = readIndexBlock(1);
  long long idxBlockId = 0;                                    // which block idxBlockNow holds
  int idxSub = 0;                                              // next chunk of that block to hand out
  // Index of this lane's row (lane < G) in the next chunk to be issued (chunks are issued in order).
  auto indexFor = [&](long long) -> long long {
    if (idxSub == chunksPerBlock) {  // uniform across the warp
      idxBlockNow = idxBlockNext;
      idxBlockNext = readIndexBlock(++idxBlockId + 1);
      idxSub = 0;
    }
    const long long idx = __shfl_sync(0xffffffffu, idxBlockNow, idxSub * G + (lane & (G - 1)));
    ++idxSub;
    return idx;
  };
  // Issues the copies of `chunk` into `stage`; returns the mask of lanes whose row is live (valid index).
  auto issue = [&](long long chunk, int stage, long long idx) -> unsigned int {
    const long long row0 = chunk * G;
    const int n = static_cast<int>(min(static_cast<long long>(G), rangeEnd - row0));
    const bool mine = lane < n;
    const bool valid = mine && idx >= 0 && idx < prm.tableRows;
    if (mine && !valid && prm.status) atomicAdd(prm.status, 1ull);
    const unsigned int live = __ballot_sync(0xffffffffu, valid);
    const unsigned int bar = gaSmemU32(&bars[stage]);
    unsigned char *stg = ring + static_cast<size_t>(stage) * stageBytes;
    const bool allLive = live == (n >= 32 ? 0xffffffffu : ((1u << n) - 1u));
    if (lane == 0) {
      const unsigned int rowsLive = __popc(live);
      // table rows of live lanes + streamed rows (whole chunk when contiguous and all live, else live rows only)
      unsigned int bytes = rowsLive * prm.rowBytes;
      for (int k = 1; k < prm.numViews; ++k)
        if (prm.slot[k] > 0) bytes += (allLive && prm.rowStrideBytes[k] == prm.rowBytes ? static_cast<unsigned int>(n) : rowsLive) * prm.rowBytes;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    }
    __syncwarp();
    if (valid) {
      const char *src = prm.table + idx * prm.tableRowStrideBytes;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(gaSmemU32(stg + lane * prm.rowBytes)), "l"(src), "r"(prm.rowBytes), "r"(bar) : "memory");
    }
    for (int k = 1; k < prm.numViews; ++k) {
      if (prm.slot[k] <= 0) continue;
      unsigned char *dst = stg + static_cast<size_t>(prm.slot[k]) * bufBytes;
      if (allLive && prm.rowStrideBytes[k] == prm.rowBytes) {
        if (lane == 0)
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(gaSmemU32(dst)), "l"(prm.vbase[k] + row0 * prm.rowStrideBytes[k]), "r"(static_cast<unsigned int>(n) * prm.rowBytes), "r"(bar) : "memory");
      } else if (valid) {
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(gaSmemU32(dst + lane * prm.rowBytes)), "l"(prm.vbase[k] + (row0 + lane) * prm.rowStrideBytes[k]), "r"(prm.rowBytes), "r"(bar) : "memory");
      }
    }
    return live;
  };

  // prologue: fill every stage
  unsigned int liveMask[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) liveMask[s] = 0;
  long long issueChunk = firstChunk;
  int issueStage = 0;
  for (int s = 0; s < S && issueChunk < numChunks; ++s) {
    const unsigned int live = issue(issueChunk, issueStage, indexFor(issueChunk));
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (q == issueStage) liveMask[q] = live;
    ++issueChunk;
    issueStage = issueStage + 1 == S ? 0 : issueStage + 1;
  }

  int stage = 0;
  unsigned int phaseBits = 0;  // bit s = parity to wait for on stage s
  bool timedOut = false;
  for (long long chunk = firstChunk; chunk < numChunks && !timedOut; ++chunk) {
    const long long row0 = chunk * G;
    const int n = static_cast<int>(min(static_cast<long long>(G), rangeEnd - row0));
    const unsigned int bar = gaSmemU32(&bars[stage]);
    const unsigned int parity = (phaseBits >> stage) & 1u;
    timedOut = !gaWaitStage(bar, parity);
    timedOut = __any_sync(0xffffffffu, timedOut);
    if (timedOut) break;
    phaseBits ^= 1u << stage;
    unsigned int live = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (q == stage) live = liveMask[q];

    // Shared-memory offsets (32-bit) of the stage's table rows and of every streamed view's rows; views that are
    // broadcast along the rows are read from global memory once per column.
    const unsigned int stg = ringU32 + static_cast<unsigned int>(stage) * stageBytes;
    unsigned int viewOff[NV];
    bool streamed[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      streamed[k] = k >= 1 && k < prm.numViews && prm.slot[k] > 0;
      viewOff[k] = stg + (streamed[k] ? static_cast<unsigned int>(prm.slot[k]) * bufBytes : 0u);
    }
    auto ldsVec = [](unsigned int addr) {
      uint4 v;
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
      return v;
    };
    auto evalVec = [&](const uint4 (&raw)[NV]) {
      Vec16<P> o;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        P vals[NV];
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const unsigned int bits = q == 0 ? raw[k].x : q == 1 ? raw[k].y : q == 2 ? raw[k].z : raw[k].w;
          vals[k] = P::fromBits(bits);
        }
        o.p[q] = B::template eval<P>(vals, prm.prog);
      }
      return o.raw();
    };
    auto loadBroadcast = [&](unsigned int col, uint4 (&bcast)[NV]) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        bcast[k] = make_uint4(0u, 0u, 0u, 0u);
        if (k >= 1 && k < prm.numViews && !streamed[k]) bcast[k] = loadKeep16(prm.vbase[k] + col * 16);
      }
    };
    if (prm.vecPerRow >= 32) {
      // a lane keeps its column(s): row-broadcast operands are read once per column, then the rows of the stage,
      // four at a time (all shared-memory loads first, then the arithmetic and the stores)
      const bool allRows = live == (n >= 32 ? 0xffffffffu : ((1u << n) - 1u));
      for (unsigned int col = lane; col < prm.vecPerRow; col += 32) {
        uint4 bcast[NV];
        loadBroadcast(col, bcast);
        unsigned int off = col * 16;                        // byte offset of (row 0, col) inside a view's rows
        char *dst = prm.out + row0 * prm.outRowStrideBytes + col * 16;
        int g = 0;
        if (allRows) {
          for (; g + 4 <= n; g += 4) {
            uint4 raw[4][NV];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
              for (int k = 0; k < NV; ++k) raw[u][k] = (k == 0 || streamed[k]) ? ldsVec(viewOff[k] + off + u * prm.rowBytes) : bcast[k];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) storeStream16(dst + u * prm.outRowStrideBytes, evalVec(raw[u]));
            off += 4 * prm.rowBytes;
            dst += 4 * prm.outRowStrideBytes;
          }
        }
        for (; g < n; ++g) {
          if ((live >> g) & 1u) {
            uint4 raw[NV];
#pragma unroll
            for (int k = 0; k < NV; ++k) raw[k] = (k == 0 || streamed[k]) ? ldsVec(viewOff[k] + off) : bcast[k];
            storeStream16(dst, evalVec(raw));
          }
          off += prm.rowBytes;
          dst += prm.outRowStrideBytes;
        }
      }
    } else {
      const unsigned int nvec = static_cast<unsigned int>(n) * prm.vecPerRow;
      for (unsigned int v = lane; v < nvec; v += 32) {
        const unsigned int g = fastDivide(v, prm.divVpr);
        const unsigned int col = v - g * prm.vecPerRow;
        if (!((live >> g) & 1u)) continue;
        uint4 bcast[NV], raw[NV];
        loadBroadcast(col, bcast);
#pragma unroll
        for (int k = 0; k < NV; ++k) raw[k] = (k == 0 || streamed[k]) ? ldsVec(viewOff[k] + v * 16) : bcast[k];
        storeStream16(prm.out + (row0 + g) * prm.outRowStrideBytes + col * 16, evalVec(raw));
      }
    }
    // every lane has finished reading the stage: refill it with the chunk S stages ahead
    __syncwarp();
    if (issueChunk < numChunks) {
      const unsigned int l2 = issue(issueChunk, issueStage, indexFor(issueChunk));
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q == issueStage) liveMask[q] = l2;
      ++issueChunk;
      issueStage = issueStage + 1 == S ? 0 : issueStage + 1;
    }
    stage = stage + 1 == S ? 0 : stage + 1;
  }
  if (timedOut) {
    // copies into the other stages may still be in flight: give each of them one more bounded wait before the
    // shared memory they target is given up
    if (lane == 0 && prm.status) atomicOr(prm.status, kGatherTimeoutFlag);
    for (int s = 0; s < S; ++s)
      if (s != stage) gaWaitStage(gaSmemU32(&bars[s]), (phaseBits >> s) & 1u);
  }
}

using KernelFn = void (*)(const GaParams);

template <class P, int BODY> KernelFn pickRowsUnroll(int unroll, bool vector) {
  if (!vector) return gatherRowsKernel<P, BODY, 2, false>;
  return unroll >= 4 ? gatherRowsKernel<P, BODY, 4, true> : unroll >= 2 ? gatherRowsKernel<P, BODY, 2, true>
                                                                        : gatherRowsKernel<P, BODY, 1, true>;
}
// Sharded tables: the bodies with a specialised chain keep it (the interpreted body costs several times the
// bandwidth-bound time even on local rows), two vectors in flight per thread.
template <class P> KernelFn pickRowsSharded(int body, bool vector) {
  if (!vector) return gatherRowsKernel<P, kBodyInterpreted, 2, false, true>;
  switch (body) {
  case kBodyCopy: return gatherRowsKernel<P, kBodyCopy, 2, true, true>;
  case kBodyMulAdd: return gatherRowsKernel<P, kBodyMulAdd, 2, true, true>;
  case kBodyAdd: return gatherRowsKernel<P, kBodyAdd, 2, true, true>;
  case kBodyMul: return gatherRowsKernel<P, kBodyMul, 2, true, true>;
  default: return gatherRowsKernel<P, kBodyInterpreted, 2, true, true>;
  }
}

template <class P> KernelFn pickRows(int body, int unroll, bool vector) {
  switch (body) {
  case kBodyCopy: return pickRowsUnroll<P, kBodyCopy>(unroll, vector);
  case kBodyMulAdd: return pickRowsUnroll<P, kBodyMulAdd>(unroll, vector);
  case kBodyAdd: return pickRowsUnroll<P, kBodyAdd>(unroll, vector);
  case kBodyMul: return pickRowsUnroll<P, kBodyMul>(unroll, vector);
  default: return pickRowsUnroll<P, kBodyInterpreted>(2, vector);
  }
}
template <class P> void (*pickStream(int body))(const GaStreamParams) {
  switch (body) {
  case kBodyCopy: return gatherRowsStreamKernel<P, kBodyCopy>;
  case kBodyMulAdd: return gatherRowsStreamKernel<P, kBodyMulAdd>;
  case kBodyAdd: return gatherRowsStreamKernel<P, kBodyAdd>;
  case kBodyMul: return gatherRowsStreamKernel<P, kBodyMul>;
  default: return gatherRowsStreamKernel<P, kBodyInterpreted>;
  }
}
template <class P> KernelFn pickCols(int body) {
  switch (body) {
  case kBodyCopy: return gatherColsKernel<P, kBodyCopy>;
  case kBodyReluAdd: return gatherColsKernel<P, kBodyReluAdd>;
  case kBodyAdd: return gatherColsKernel<P, kBodyAdd>;
  default: return gatherColsKernel<P, kBodyInterpreted>;
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

} // namespace

int launchGather(const GatherLaunch &l, cudaStream_t stream, int *launched) {
  if (launched) *launched = 0;
  if (l.rows == 0 || l.cols == 0) return cudaSuccess;
  if (l.numViews < 1 || l.numViews > kMaxViews) return cudaErrorInvalidValue;
  const int eb = elemBytes(l.elemType);
  const int vecElems = 16 / eb;

  GaParams p = {};
  p.table = static_cast<const char *>(l.table);
  p.tableRows = l.tableRows;
  p.tableCols = l.tableCols;
  p.tableRowStride = l.tableRowStride;
  p.indices = l.indices;
  p.index64 = l.indexType == kI64 ? 1 : 0;
  for (int k = 1; k < l.numViews; ++k) {
    p.vbase[k] = static_cast<const char *>(l.views[k].base);
    p.rowStride[k] = l.views[k].rowStride;
    p.colStride[k] = static_cast<int>(l.views[k].colStride);
  }
  p.numViews = l.numViews;
  p.out = static_cast<char *>(l.out);
  p.outRowStride = l.outRowStride;
  p.status = l.status;
  p.prog = l.body;

  bool shardsAligned = true;
  if (l.numShards > 0) {
    if (l.axis != 0 || l.numShards > kMaxTableShards || l.rowsPerShard <= 0 || l.tableRows >= (1ll << 32) ||
        l.rowsPerShard * l.numShards < l.tableRows)
      return cudaErrorInvalidValue;
    for (int sh = 0; sh < l.numShards; ++sh) {
      if (!l.tableShards[sh]) return cudaErrorInvalidValue;
      p.shardBase[sh] = static_cast<const char *>(l.tableShards[sh]);
      shardsAligned = shardsAligned && aligned16(l.tableShards[sh]);
    }
    p.rowsPerShard = l.rowsPerShard;
    p.divRowsPerShard = makeFastDiv(static_cast<unsigned int>(std::min<int64_t>(l.rowsPerShard, 0xffffffffll)));
  }

  int threads = l.ctaThreads > 0 ? l.ctaThreads : 128;
  threads = std::max(32, std::min(512, (threads / 32) * 32));
  const int body = matchBody(l.body, l.numViews);
  KernelFn fn;
  int64_t totalVec, numTiles;
  if (l.axis == 0) {
    bool vector = l.cols % vecElems == 0 && (l.numShards > 0 ? shardsAligned : aligned16(l.table)) && l.tableRowStride % vecElems == 0 &&
                  aligned16(l.out) && l.outRowStride % vecElems == 0;
    for (int k = 1; k < l.numViews && vector; ++k) {
      if (l.views[k].colStride == 1) vector = aligned16(l.views[k].base) && l.views[k].rowStride % vecElems == 0;
      else if (l.views[k].colStride != 0) vector = false;
    }
    // Bulk-copy staged kernel, on request only: aligned rows of 128 bytes to 16 KB, every other view either one
    // row per output row or one row for all, enough chunks to give every warp of the machine a few.
    if (vector && l.stagedCopies && l.numShards == 0) {
      const int64_t rowBytes = l.cols * eb;
      int numStreamed = 0;
      bool eligible = rowBytes >= 128 && rowBytes <= 16384 && (l.tableRowStride * eb) % 16 == 0 && (l.outRowStride * eb) % 16 == 0;
      GaStreamParams sp = {};
      for (int k = 1; k < l.numViews && eligible; ++k) {
        sp.slot[k] = -1;
        sp.vbase[k] = static_cast<const char *>(l.views[k].base);
        sp.rowStrideBytes[k] = l.views[k].rowStride * eb;
        if (l.views[k].colStride != 1) eligible = false;
        else if (l.views[k].rowStride != 0) {
          if (++numStreamed > kMaxStreamedViews) eligible = false;
          sp.slot[k] = numStreamed;
        }
      }
      int device = 0;
      cudaGetDevice(&device);
      int sms = 0;
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
      int warps = l.streamWarps > 0 ? std::max(1, std::min(16, l.streamWarps)) : 8;
      int G = l.streamRows > 0 ? l.streamRows : static_cast<int>(std::max<int64_t>(1, 4096 / rowBytes));
      G = std::max(1, std::min(32, G));
      while (G & (G - 1)) G &= G - 1;  // a power of two, so that blocks of 32 indices split into whole chunks
      int S = l.streamStages > 0 ? l.streamStages : 3;
      S = std::max(2, std::min(8, S));
      auto smemFor = [&](int w, int st, int g) {
        return static_cast<size_t>(w) * st * (1 + numStreamed) * g * rowBytes + static_cast<size_t>(w) * st * sizeof(unsigned long long);
      };
      while (smemFor(warps, S, G) > 200 * 1024 && S > 2) --S;
      while (smemFor(warps, S, G) > 200 * 1024 && G > 1) G /= 2;
      while (smemFor(warps, S, G) > 200 * 1024 && warps > 1) warps /= 2;
      const int64_t chunks = (l.rows + G - 1) / G;
      if (eligible && smemFor(warps, S, G) <= 200 * 1024 && chunks >= static_cast<int64_t>(sms) * warps * 2 && l.rows < (1ll << 40)) {
        sp.table = static_cast<const char *>(l.table);
        sp.tableRows = l.tableRows;
        sp.tableRowStrideBytes = l.tableRowStride * eb;
        sp.indices = l.indices;
        sp.index64 = l.indexType == kI64 ? 1 : 0;
        sp.numViews = l.numViews;
        sp.numStreamed = numStreamed;
        sp.out = static_cast<char *>(l.out);
        sp.outRowStrideBytes = l.outRowStride * eb;
        sp.rows = l.rows;
        sp.rowBytes = static_cast<unsigned int>(rowBytes);
        sp.vecPerRow = static_cast<unsigned int>(rowBytes / 16);
        sp.divVpr = makeFastDiv(sp.vecPerRow);
        sp.rowsPerStage = G;
        sp.stages = S;
        sp.status = l.status;
        sp.prog = l.body;
        using StreamFn = void (*)(const GaStreamParams);
        StreamFn sfn = l.elemType == kF32 ? pickStream<PackF32>(body) : l.elemType == kF16 ? pickStream<PackF16>(body) : pickStream<PackBF16>(body);
        const size_t smem = smemFor(warps, S, G);
        cudaError_t ae = cudaFuncSetAttribute(sfn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (ae != cudaSuccess) return ae;
        const int64_t groups = (chunks + warps - 1) / warps;
        int64_t sgrid = l.gridBlocks > 0 ? l.gridBlocks : sms;
        sgrid = std::max<int64_t>(1, std::min<int64_t>(sgrid, groups));
        launchOrdinary(sfn, static_cast<unsigned int>(sgrid), warps * 32, smem, stream, sp);
        if (launched) *launched = 1;
        return cudaGetLastError();
      }
    }
    int unroll = l.unroll > 0 ? l.unroll : 1;
    unroll = unroll >= 4 ? 4 : unroll >= 2 ? 2 : 1;
    if (!vector || body == kBodyInterpreted || (body != kBodyCopy && body != kBodyMulAdd && body != kBodyAdd && body != kBodyMul))
      unroll = 2;
    const int64_t vecPerRow = l.cols / (vector ? vecElems : 1);
    totalVec = l.rows * vecPerRow;
    if (totalVec >= (1ll << 32) - (1 << 20) || vecPerRow >= (1ll << 31)) return cudaErrorInvalidValue;
    p.vecPerRow = static_cast<unsigned int>(vecPerRow);
    fn = l.elemType == kF32 ? pickRows<PackF32>(body, unroll, vector)
         : l.elemType == kF16 ? pickRows<PackF16>(body, unroll, vector)
                              : pickRows<PackBF16>(body, unroll, vector);
    if (l.numShards > 0) {
      unroll = 2;
      fn = l.elemType == kF32 ? pickRowsSharded<PackF32>(body, vector)
           : l.elemType == kF16 ? pickRowsSharded<PackF16>(body, vector)
                                : pickRowsSharded<PackBF16>(body, vector);
    }
    const int64_t tileVecs = static_cast<int64_t>(threads) * unroll;
    numTiles = (totalVec + tileVecs - 1) / tileVecs;
  } else {
    totalVec = l.rows * l.cols;
    if (totalVec >= (1ll << 32) - (1 << 20) || l.cols >= (1ll << 31)) return cudaErrorInvalidValue;
    p.vecPerRow = static_cast<unsigned int>(l.cols);
    fn = l.elemType == kF32 ? pickCols<PackF32>(body) : l.elemType == kF16 ? pickCols<PackF16>(body) : pickCols<PackBF16>(body);
    numTiles = (totalVec + threads - 1) / threads;
  }
  p.totalVec = static_cast<unsigned int>(totalVec);
  p.divVpr = makeFastDiv(p.vecPerRow);
  int64_t grid = l.gridBlocks > 0 ? l.gridBlocks : numTiles;
  grid = std::max<int64_t>(1, std::min<int64_t>(grid, numTiles));
  launchOrdinary(fn, static_cast<unsigned int>(grid), threads, 0, stream, p);
  if (launched) *launched = 1;
  return cudaGetLastError();
}

} // namespace kernels
} // namespace afir
