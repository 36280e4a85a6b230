// Broadcast + elementwise + row reduction groups: out[m] = sum_n body(views)(m, n)
// (the [parallel, reduction] linalg.generic class, lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:244-748;
// zero-initialised accumulator per :508-521; 16-bit inputs are summed as f32 and cast back,
// lib/Target/CannKernel/CannTranslation.cpp:2446-2461).
//
// HBM-bound streaming read.  L threads cooperate on one row (L = 32..CTA size), each keeping four
// 16-byte loads per view in flight; warp-shuffle tree, then a shared-memory tree across warps, f32
// accumulators throughout.  Short-and-wide problems split each row into column slices whose partial
// sums go to the workspace and are added in slice order by a second kernel (deterministic).
#include "kernels/ew_common.cuh"

#include <algorithm>
#include <cstdio>
#include <mutex>

namespace afir {
namespace kernels {
namespace {

struct RrParams {
  const char *vbase[kMaxViews];
  long long rowStride[kMaxViews];
  int colStride[kMaxViews];
  int numViews;
  long long rows;
  unsigned int vecPerRow;    // vectors (or elements) per full row
  unsigned int vecPerSlice;  // vectors per column slice
  int slices;
  int lanesPerRow;           // power of two, 32..blockDim.x
  float *partial;            // [rows, slices] when slices > 1
  void *out;
  BodyProgram prog;
  RowReduceExchange xchg;    // world > 0: the sums are partial and go to every rank's mailbox
};

template <class P> __device__ __forceinline__ void storeSum(void *out, long long row, float v);
template <> __device__ __forceinline__ void storeSum<PackF32>(void *out, long long row, float v) {
  static_cast<float *>(out)[row] = v;
}
template <> __device__ __forceinline__ void storeSum<PackF16>(void *out, long long row, float v) {
  static_cast<__half *>(out)[row] = __float2half_rn(v);
}
template <> __device__ __forceinline__ void storeSum<PackBF16>(void *out, long long row, float v) {
  static_cast<__nv_bfloat16 *>(out)[row] = __float2bfloat16_rn(v);
}

// ---- exchange of partial sums between GPUs (the reduced axis is sharded) ----------------------------------
// A mailbox entry is eight bytes, {f32 partial sum, epoch}, written with ONE 8-byte store, so value and "it has
// arrived" travel together and a reader never sees half an entry: no flags, no fences.  Each row's partial sum
// is stored into every rank's mailbox (plain stores over NVLink; the own mailbox is a local store).  A reader
// polls an entry until its epoch is the call's, then adds the world's partial sums in rank order, so all ranks
// produce the same bits.  Who reads: in the persistent staged kernel the warp that sent a row reads that row
// one row later (the NVLink latency hides behind the next row's stream; every rank walks its rows in the same
// order and always sends before it reads, so no rank waits for something that itself waits); in the plain
// kernel, whose CTAs need not all be resident, the last CTA to finish reads all rows.  Every wait is bounded:
// after 2 s the status word is set, the remaining rows stay unwritten and the context remains usable.
constexpr unsigned long long kExchangeWaitLimitNs = 2000000000ull;

__device__ __forceinline__ void sendPartial(const RowReduceExchange &x, long long row, float v) {
  const unsigned long long entry = (static_cast<unsigned long long>(x.epoch) << 32) | __float_as_uint(v);
  for (int p = 0; p < x.world; ++p)
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(x.peerEntries[p] + row), "l"(entry) : "memory");
}

__device__ __forceinline__ unsigned long long peekEntry(const unsigned long long *entry) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(entry) : "memory");
  return w;
}

// Polls until the entry carries `epoch`; false when the time ran out.
__device__ __forceinline__ bool awaitEntry(const unsigned long long *entry, unsigned int epoch, unsigned long long &w) {
  unsigned long long t0 = 0;
  unsigned int spins = 0;
  while (true) {
    w = peekEntry(entry);
    if (static_cast<unsigned int>(w >> 32) == epoch) return true;
    if (++spins > 1000u) __nanosleep(100);
    if ((spins & 63u) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > kExchangeWaitLimitNs) return false;
    }
  }
}

// One warp finishes one row: lane p fetches rank p's partial sum, all lanes add them in rank order.
template <class P> __device__ __forceinline__ bool finishRowByWarp(const RowReduceExchange &x, void *out, long long row, int lane) {
  unsigned long long w = 0;
  bool ok = true;
  if (lane < x.world) ok = awaitEntry(x.myEntries + lane * x.slotStride + row, x.epoch, w);
  ok = __all_sync(0xffffffffu, ok) != 0;
  float t = 0.f;
  for (int p = 0; p < x.world; ++p) t += __uint_as_float(__shfl_sync(0xffffffffu, static_cast<unsigned int>(w), p));
  if (ok && lane == 0) storeSum<P>(out, row, t);
  return ok;
}

// Plain kernel: the last CTA to finish reads every row.
template <class P> __device__ __noinline__ void exchangeTail(const RowReduceExchange &x, void *out, long long rows) {
  __shared__ int lastCta;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    lastCta = atomicAdd(x.doneCounter, 1u) == gridDim.x - 1u;
  }
  __syncthreads();
  if (!lastCta) return;
  if (threadIdx.x == 0) *x.doneCounter = 0;  // the next launch on this stream counts from zero
  bool ok = true;
  constexpr int kRowsInFlight = 4;
  for (long long r0 = threadIdx.x; r0 < rows && ok; r0 += static_cast<long long>(kRowsInFlight) * blockDim.x) {
    float t[kRowsInFlight];
#pragma unroll
    for (int u = 0; u < kRowsInFlight; ++u) t[u] = 0.f;
    for (int p = 0; p < x.world && ok; ++p) {
      const unsigned long long *slot = x.myEntries + p * x.slotStride;
      unsigned long long w[kRowsInFlight];
#pragma unroll
      for (int u = 0; u < kRowsInFlight; ++u) {  // all four loads leave before the first is looked at
        const long long row = r0 + static_cast<long long>(u) * blockDim.x;
        w[u] = row < rows ? peekEntry(slot + row) : 0ull;
      }
#pragma unroll
      for (int u = 0; u < kRowsInFlight; ++u) {
        const long long row = r0 + static_cast<long long>(u) * blockDim.x;
        if (row < rows && static_cast<unsigned int>(w[u] >> 32) != x.epoch) ok = ok && awaitEntry(slot + row, x.epoch, w[u]);
        t[u] += __uint_as_float(static_cast<unsigned int>(w[u]));
      }
    }
    if (ok) {
#pragma unroll
      for (int u = 0; u < kRowsInFlight; ++u) {
        const long long row = r0 + static_cast<long long>(u) * blockDim.x;
        if (row < rows) storeSum<P>(out, row, t[u]);
      }
    }
  }
  if (!ok) atomicExch(x.status, 1u);
}

template <class P, int BODY, bool VECTOR, bool XCHG = false>
__global__ void __launch_bounds__(512) rowReduceKernel(const __grid_constant__ RrParams prm) {
  using B = Body<BODY>;
  constexpr int NV = B::kViews;
  constexpr int kElems = VECTOR ? Vec16<P>::kElems : 1;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
  constexpr int kBatch = 4;
  __shared__ float warpSums[16];

  const int L = prm.lanesPerRow;
  const int rowsPerCta = blockDim.x / L;
  const int sub = threadIdx.x / L;   // which row of this CTA
  const int lane = threadIdx.x % L;  // position within the row team
  const long long rowGroups = (prm.rows + rowsPerCta - 1) / rowsPerCta;
  const long long work = rowGroups * prm.slices;

  for (long long w = blockIdx.x; w < work; w += gridDim.x) {
    const long long row = (w / prm.slices) * rowsPerCta + sub;
    const int slice = static_cast<int>(w % prm.slices);
    const bool rowLive = row < prm.rows;
    const unsigned int vBegin = static_cast<unsigned int>(slice) * prm.vecPerSlice;
    const unsigned int vEnd = min(vBegin + prm.vecPerSlice, prm.vecPerRow);

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (rowLive) {
      const char *rowBase[NV];
      uint4 bcast[NV];
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        rowBase[k] = nullptr;
        bcast[k] = make_uint4(0u, 0u, 0u, 0u);
        if (k < prm.numViews) {
          rowBase[k] = prm.vbase[k] + row * prm.rowStride[k] * kElemBytes;
          if (prm.colStride[k] == 0) {
            const unsigned int s = P::splat(rowBase[k]).bits();
            bcast[k] = make_uint4(s, s, s, s);
          }
        }
      }
      for (unsigned int v0 = vBegin + lane; v0 < vEnd; v0 += kBatch * L) {
        uint4 raw[kBatch][NV];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const unsigned int v = v0 + u * L;
#pragma unroll
          for (int k = 0; k < NV; ++k) {
            raw[u][k] = bcast[k];
            if (k < prm.numViews && prm.colStride[k] != 0 && v < vEnd) {
              const char *src = rowBase[k] + static_cast<long long>(v) * kElems * prm.colStride[k] * kElemBytes;
              if (VECTOR) raw[u][k] = loadStream16(src);
              else {
                const unsigned int s = P::splat(src).bits();
                raw[u][k] = make_uint4(s, s, s, s);
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          if (VECTOR && BODY == kBodyInterpreted) {
            if (v0 + u * L < vEnd) {  // the interpreted body decodes its ops once per 16-byte vector
              const uint4 y16 = evalVector16<BODY, P, NV>(raw[u], prm.prog);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const P y = P::fromBits(comp(y16, q));
                acc[q] += y.lane(0);
                if (P::kLanes == 2) acc[q] += y.lane(1);
              }
            }
          } else if (v0 + u * L < vEnd) {
#pragma unroll
            for (int q = 0; q < (VECTOR ? 4 : 1); ++q) {
              P vals[NV];
#pragma unroll
              for (int k = 0; k < NV; ++k) {
                const unsigned int bits = q == 0 ? raw[u][k].x : q == 1 ? raw[u][k].y : q == 2 ? raw[u][k].z : raw[u][k].w;
                vals[k] = P::fromBits(bits);
              }
              const P y = B::template eval<P>(vals, prm.prog);
              acc[q] += y.lane(0);
              if (VECTOR && P::kLanes == 2) acc[q] += y.lane(1);
            }
          }
        }
      }
    }
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    // team reduction: shuffle tree inside each warp, then a shared-memory tree across the team's warps
    const int width = L < 32 ? L : 32;
    for (int off = width / 2; off > 0; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off, width);
    if (L > 32) {
      const int warp = threadIdx.x >> 5;
      const int warpsPerTeam = L >> 5;
      __syncthreads();
      if ((threadIdx.x & 31) == 0) warpSums[warp] = sum;
      __syncthreads();
      if (lane == 0) {
        float t = 0.f;
        for (int i = 0; i < warpsPerTeam; ++i) t += warpSums[sub * warpsPerTeam + i];
        sum = t;
      }
    }
    if (lane == 0 && rowLive) {
      if (XCHG) sendPartial(prm.xchg, row, sum);
      else if (prm.slices > 1) prm.partial[row * prm.slices + slice] = sum;
      else storeSum<P>(prm.out, row, sum);
    }
  }
  if constexpr (XCHG) exchangeTail<P>(prm.xchg, prm.out, prm.rows);
}

// ---- bulk-copy staged variant -------------------------------------------------------------------------
// For long rows with one streamed operand.  Registers cap how many bytes plain loads keep in flight
// (about 90 KB per SM at the occupancy the kernel above reaches); here every warp owns a ring of
// `stages` x `chunkBytes` shared-memory stages filled by cp.async.bulk (the TMA engine), so up to 192 KB per SM
// are in flight regardless of registers.  A warp walks whole rows: lane 0 refills a stage right after
// the warp has consumed it (program order + __syncwarp make the stage free, so only "full" barriers
// exist), lanes read the stage with conflict-free 16-byte shared loads, accumulate in f32 and finish
// each row with a shuffle tree.  No block-level synchronisation at all.
// Waits on the "full" barriers are bounded (2 s): on timeout the warp records g_rowReduceStatus and returns.
// Defaults from a sweep on B200 (8192 x 8192 f32): two 8 KB stages per warp, 8 warps per SM reach 97 % of
// the measured copy bandwidth; deeper rings put more independent streams in flight and lose DRAM locality.
constexpr int kStreamChunkBytesDefault = 8192;
constexpr int kStreamStagesDefault = 2;
constexpr int kStreamWarpsDefault = 8;
constexpr int kStreamMaxChunkBytes = 16384;
constexpr unsigned long long kStreamWaitLimitNs = 2000000000ull;
__device__ unsigned int g_rowReduceStatus = 0;

struct RrStreamParams {
  const char *stream;            // the streamed view
  long long streamRowStride;     // elements
  const char *bcast[kMaxViews];  // broadcast views (column stride 0), null where unused
  long long bcastRowStride[kMaxViews];
  int streamViewIndex;           // position of the streamed view among the body's views
  int numViews;
  long long rows;
  unsigned int rowBytes;         // multiple of 16
  int stages;                    // ring depth per warp
  unsigned int chunkBytes;       // multiple of 512
  void *out;
  BodyProgram prog;
  RowReduceExchange xchg;        // world > 0: the sums are partial and go to every rank's mailbox
};

__device__ __forceinline__ unsigned int smemU32(const void *p) { return static_cast<unsigned int>(__cvta_generic_to_shared(p)); }

template <class P, int BODY, bool XCHG = false>
__global__ void __launch_bounds__(512, 1) rowReduceStreamKernel(const __grid_constant__ RrStreamParams prm) {
  using B = Body<BODY>;
  constexpr int NV = B::kViews;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
  extern __shared__ __align__(128) unsigned char streamSmem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kStreamWarps = blockDim.x >> 5;
  const int kStreamStages = prm.stages;
  const unsigned int kStreamChunkBytes = prm.chunkBytes;
  unsigned char *ring = streamSmem + static_cast<size_t>(warp) * kStreamStages * kStreamChunkBytes;
  unsigned long long *fullBars = reinterpret_cast<unsigned long long *>(streamSmem + static_cast<size_t>(kStreamWarps) * kStreamStages * kStreamChunkBytes) + warp * kStreamStages;

  if (lane == 0) {
    for (int s = 0; s < kStreamStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemU32(&fullBars[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  const long long totalWarps = static_cast<long long>(gridDim.x) * kStreamWarps;
  const long long firstRow = static_cast<long long>(blockIdx.x) * kStreamWarps + warp;
  const unsigned int chunksPerRow = (prm.rowBytes + kStreamChunkBytes - 1) / kStreamChunkBytes;

  // producer cursor (lane 0 only uses it)
  long long prodRow = firstRow;
  unsigned int prodChunk = 0;
  auto issue = [&](int stage) {
    const unsigned int off = prodChunk * kStreamChunkBytes;
    const unsigned int bytes = min(kStreamChunkBytes, prm.rowBytes - off);
    const char *src = prm.stream + prodRow * prm.streamRowStride * kElemBytes + off;
    const unsigned int bar = smemU32(&fullBars[stage]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smemU32(ring + stage * kStreamChunkBytes)), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
    if (++prodChunk == chunksPerRow) { prodChunk = 0; prodRow += totalWarps; }
  };
  if (lane == 0)
    for (int s = 0; s < kStreamStages && prodRow < prm.rows; ++s) issue(s);

  auto loadBcast = [&](long long row, unsigned int (&dst)[NV]) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      dst[k] = 0u;
      if (k < prm.numViews && k != prm.streamViewIndex && row < prm.rows)
        dst[k] = P::splat(prm.bcast[k] + row * prm.bcastRowStride[k] * kElemBytes).bits();
    }
  };

  int stage = 0;
  unsigned int phase = 0;
  unsigned int bcastNow[NV], bcastNext[NV];
  loadBcast(firstRow, bcastNow);
  long long sentRow = -1;  // exchange: the row this warp has sent but not yet finished
  bool peersAnswer = true;  // exchange: false once a wait for another rank ran out (the warp then only drains its stream)
  for (long long row = firstRow; row < prm.rows; row += totalWarps) {
    loadBcast(row + totalWarps, bcastNext);  // one row ahead: its latency hides behind this row's stream
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (unsigned int chunk = 0; chunk < chunksPerRow; ++chunk) {
      // bounded wait for the stage
      const unsigned int bar = smemU32(&fullBars[stage]);
      unsigned int done = 0, spins = 0;
      unsigned long long t0 = 0;
      while (true) {
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(phase) : "memory");
        if (done) break;
        if ((++spins & 255u) == 0) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (t0 == 0) t0 = now;
          else if (now - t0 > kStreamWaitLimitNs) {
            atomicCAS(&g_rowReduceStatus, 0u, 1u);
            return;  // nothing of this warp's is in flight on a barrier that never completed beyond this ring
          }
        }
      }
      const unsigned int bytes = min(kStreamChunkBytes, prm.rowBytes - chunk * kStreamChunkBytes);
      const unsigned int nvec = bytes >> 4;
      const unsigned char *stg = ring + stage * kStreamChunkBytes;
#pragma unroll 4
      for (unsigned int v = lane; v < nvec; v += 32) {
        {
          const uint4 raw = *reinterpret_cast<const uint4 *>(stg + v * 16);
          if constexpr (BODY == kBodyInterpreted) {
            uint4 all[NV];
#pragma unroll
            for (int k = 0; k < NV; ++k)
              all[k] = k == prm.streamViewIndex ? raw : make_uint4(bcastNow[k], bcastNow[k], bcastNow[k], bcastNow[k]);
            const uint4 y16 = evalVector16<BODY, P, NV>(all, prm.prog);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const P y = P::fromBits(comp(y16, q));
              acc[q] += y.lane(0);
              if (P::kLanes == 2) acc[q] += y.lane(1);
            }
          } else
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const unsigned int bits = q == 0 ? raw.x : q == 1 ? raw.y : q == 2 ? raw.z : raw.w;
            P vals[NV];
#pragma unroll
            for (int k = 0; k < NV; ++k) vals[k] = P::fromBits(k == prm.streamViewIndex ? bits : bcastNow[k]);
            const P y = B::template eval<P>(vals, prm.prog);
            acc[q] += y.lane(0);
            if (P::kLanes == 2) acc[q] += y.lane(1);
          }
        }
      }
      __syncwarp();
      if (lane == 0 && prodRow < prm.rows) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(stage);
      }
      if (++stage == kStreamStages) { stage = 0; phase ^= 1u; }
    }
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off);
    if constexpr (XCHG) {
      if (lane == 0) sendPartial(prm.xchg, row, sum);
      if (sentRow >= 0 && peersAnswer) peersAnswer = finishRowByWarp<P>(prm.xchg, prm.out, sentRow, lane);
      sentRow = row;
    } else {
      if (lane == 0) storeSum<P>(prm.out, row, sum);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) bcastNow[k] = bcastNext[k];
  }
  if constexpr (XCHG) {
    if (sentRow >= 0 && peersAnswer) peersAnswer = finishRowByWarp<P>(prm.xchg, prm.out, sentRow, lane);
    if (!peersAnswer && lane == 0) atomicExch(prm.xchg.status, 1u);
  }
}

template <class P>
__global__ void rowReduceFinalizeKernel(const float *__restrict__ partial, void *out, long long rows, int slices) {
  const long long row = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float t = 0.f;
  for (int s = 0; s < slices; ++s) t += partial[row * slices + s];
  storeSum<P>(out, row, t);
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

int launchRowReduce(const RowReduceLaunch &l, cudaStream_t stream, int *launched) {
  if (launched) *launched = 0;
  if (l.rows == 0) return cudaSuccess;
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

  int threads = l.ctaThreads > 0 ? l.ctaThreads : 128;
  threads = threads >= 512 ? 512 : threads >= 256 ? 256 : threads >= 128 ? 128 : threads >= 64 ? 64 : 32;
  // team size: enough lanes that each does about one batch of four vectors, at least a warp
  int lanes = 32;
  while (lanes < threads && static_cast<int64_t>(lanes) * 4 < vecPerSlice) lanes <<= 1;
  if (l.teamLanes >= 32) {
    lanes = 32;
    while (lanes * 2 <= l.teamLanes && lanes * 2 <= threads) lanes <<= 1;
  }

  RrParams p = {};
  for (int k = 0; k < l.numViews; ++k) {
    p.vbase[k] = static_cast<const char *>(l.views[k].base);
    p.rowStride[k] = l.views[k].rowStride;
    p.colStride[k] = static_cast<int>(l.views[k].colStride);
  }
  p.numViews = l.numViews;
  p.rows = l.rows;
  p.vecPerRow = static_cast<unsigned int>(vecPerRow);
  p.vecPerSlice = static_cast<unsigned int>(vecPerSlice);
  p.slices = slices;
  p.lanesPerRow = lanes;
  p.partial = static_cast<float *>(l.workspace);
  p.out = l.out;
  p.prog = l.body;
  if (l.exchange) p.xchg = *l.exchange;

  const int body = matchBody(l.body, l.numViews);
  // Long rows with exactly one streamed operand and enough rows to occupy every warp of the machine:
  // the bulk-copy staged kernel.
  if (vector && slices == 1 && !l.forcePlainLoads) {
    int streamed = -1, numStreamed = 0;
    for (int k = 0; k < l.numViews; ++k)
      if (l.views[k].colStride == 1) { streamed = k; ++numStreamed; }
    int device = 0;
    cudaGetDevice(&device);
    const int sms = deviceSmCount(device);
    const int64_t rowBytes = l.cols * eb;
    int sWarps = l.ctaThreads >= 64 ? std::min(16, l.ctaThreads / 32) : kStreamWarpsDefault;
    int sStages = l.streamStages > 0 ? std::min(32, l.streamStages) : kStreamStagesDefault;
    unsigned int sChunk = l.streamChunkBytes > 0 ? static_cast<unsigned int>(std::min(kStreamMaxChunkBytes, (l.streamChunkBytes / 512) * 512))
                                                 : static_cast<unsigned int>(kStreamChunkBytesDefault);
    if (l.streamChunkBytes <= 0 && rowBytes < 2 * static_cast<int64_t>(sChunk))  // shorter rows: at least two chunks per row
      sChunk = static_cast<unsigned int>(std::max<int64_t>(512, (rowBytes / 2 / 512) * 512));
    if (sChunk < 512) sChunk = 512;
    while (static_cast<size_t>(sWarps) * sStages * sChunk > 200 * 1024 && sStages > 2) --sStages;
    const int kStreamWarps = sWarps;
    if (numStreamed == 1 && rowBytes >= 2 * static_cast<int64_t>(sChunk) && rowBytes < (1ll << 31) &&
        l.rows >= static_cast<int64_t>(sms) * kStreamWarps) {
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
      sp.rowBytes = static_cast<unsigned int>(rowBytes);
      sp.stages = sStages;
      sp.chunkBytes = sChunk;
      sp.out = l.out;
      sp.prog = l.body;
      if (l.exchange) sp.xchg = *l.exchange;
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
      const size_t smem = static_cast<size_t>(kStreamWarps) * sStages * sChunk + static_cast<size_t>(kStreamWarps) * sStages * sizeof(unsigned long long);
      cudaError_t ae = cudaFuncSetAttribute(sfn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (ae != cudaSuccess) return ae;
      const int64_t rowGroups = (l.rows + kStreamWarps - 1) / kStreamWarps;
      int64_t sgrid = l.gridBlocks > 0 ? l.gridBlocks : sms;
      sgrid = std::max<int64_t>(1, std::min<int64_t>(sgrid, rowGroups));
      if (l.exchange) sgrid = std::min<int64_t>(sgrid, sms);  // warps that wait for other ranks: one CTA per SM, all resident
      sfn<<<static_cast<unsigned int>(sgrid), kStreamWarps * 32, smem, stream>>>(sp);
      if (launched) *launched = 1;
      return cudaGetLastError();
    }
  }
  KernelFn fn;
  if (l.elemType == kF32) fn = vector ? pickBody<PackF32, true>(body) : pickBody<PackF32, false>(body);
  else if (l.elemType == kF16) fn = vector ? pickBody<PackF16, true>(body) : pickBody<PackF16, false>(body);
  else fn = vector ? pickBody<PackBF16, true>(body) : pickBody<PackBF16, false>(body);
  if (l.exchange) {
    if (l.elemType == kF32) fn = vector ? pickBodyExchange<PackF32, true>(body) : pickBodyExchange<PackF32, false>(body);
    else if (l.elemType == kF16) fn = vector ? pickBodyExchange<PackF16, true>(body) : pickBodyExchange<PackF16, false>(body);
    else fn = vector ? pickBodyExchange<PackBF16, true>(body) : pickBodyExchange<PackBF16, false>(body);
  }

  const int rowsPerCta = threads / lanes;
  const int64_t work = ((l.rows + rowsPerCta - 1) / rowsPerCta) * slices;
  int64_t grid = l.gridBlocks > 0 ? l.gridBlocks : work;
  grid = std::max<int64_t>(1, std::min<int64_t>(grid, std::min<int64_t>(work, 0x7fffffff)));
  fn<<<static_cast<unsigned int>(grid), threads, 0, stream>>>(p);
  int n = 1;
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess && slices > 1) {
    const int ft = 256;
    const unsigned int fg = static_cast<unsigned int>((l.rows + ft - 1) / ft);
    if (l.elemType == kF32) rowReduceFinalizeKernel<PackF32><<<fg, ft, 0, stream>>>(p.partial, l.out, l.rows, slices);
    else if (l.elemType == kF16) rowReduceFinalizeKernel<PackF16><<<fg, ft, 0, stream>>>(p.partial, l.out, l.rows, slices);
    else rowReduceFinalizeKernel<PackBF16><<<fg, ft, 0, stream>>>(p.partial, l.out, l.rows, slices);
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
