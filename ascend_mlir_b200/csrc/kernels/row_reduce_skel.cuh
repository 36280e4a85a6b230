// Device side of the row-reduction kernels (out[m] = sum_n body(views)(m, n), f32 accumulation): launch records,
// the exchange of partial sums between GPUs, the team-per-row loop, the bulk-copy staged loop and the finalize
// step, as function templates over the fused body.  The prebuilt kernels instantiate them with the straight-line
// bodies and the interpreter; a kernel generated for one fused group instantiates them with that group's body.
// (Also compiled at run time by NVRTC: no host headers here.)
#pragma once

#include "kernels/ew_common.cuh"

namespace afir {
namespace kernels {

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
#ifdef AFIR_HAVE_F16
template <> __device__ __forceinline__ void storeSum<PackF16>(void *out, long long row, float v) {
  static_cast<__half *>(out)[row] = __float2half_rn(v);
}
#endif
#ifdef AFIR_HAVE_BF16
template <> __device__ __forceinline__ void storeSum<PackBF16>(void *out, long long row, float v) {
  static_cast<__nv_bfloat16 *>(out)[row] = __float2bfloat16_rn(v);
}
#endif

// ---- exchange of partial sums between GPUs (the reduced axis is sharded) ----------------------------------
// A mailbox entry is eight bytes, {f32 partial sum, epoch}, written with ONE 8-byte store, so value and "it has
// arrived" travel together and a reader never sees half an entry: no flags, no fences.  Each row's partial sum
// is stored into every rank's mailbox (plain stores over NVLink; the own mailbox is a local store).  A reader
// polls an entry until its epoch is the call's, then adds the world's partial sums in rank order, so all ranks
// produce the same bits.  Who reads: in the persistent staged kernel the warp that sent a row reads it several
// rows later, a group of rows at a time with one lane per (row, rank) entry, so that neither the NVLink latency
// nor the round trip of a poll stands between two rows of its stream (every rank walks its rows in the same
// order and a send never waits, so no rank waits for something that itself waits); in the plain kernel, whose
// CTAs need not all be resident, the last CTA to finish reads all rows.  Every wait is bounded: after 2 s the
// status word is set, the remaining rows stay unwritten and the context remains usable.
constexpr unsigned long long kExchangeWaitLimitNs = 2000000000ull;

// The call number is kept on the device in one 64-bit word, {completed calls : arrivals of the running launch}.
// Each CTA of a launch takes a ticket with ONE atomic add (per CTA, not per warp: a thousand warps adding to one
// word at kernel start were measured to cost over a microsecond).  The high half tells it the running call's
// number (one more than the completed calls; 0 is skipped, it is what an untouched entry holds, and 2 follows
// 2^32 - 1 so that the halves keep alternating), the low half its arrival index.  The last CTA to arrive moves the
// word on to {this call : 0}; by then every CTA of the launch has its number, and the next launch on the stream
// starts from the new word.  Nothing else of a launch reads the word.
__device__ __forceinline__ unsigned long long takeExchangeTicket(const RowReduceExchange &in) {
  return atomicAdd(in.callWord, 1ull);
}

// The running call's view of the exchange: its number and the pointers of its half of the mailbox.
__device__ __forceinline__ RowReduceExchange resolveExchange(const RowReduceExchange &in, unsigned long long ticket) {
  RowReduceExchange x = in;
  unsigned int e = static_cast<unsigned int>(ticket >> 32) + 1u;
  if (e == 0u) e = 2u;
  x.epoch = e;
  const long long shift = (e & 1u) ? in.halfStride : 0ll;
#pragma unroll
  for (int p = 0; p < kMaxExchangeRanks; ++p) x.peerEntries[p] = in.peerEntries[p] + shift;
  x.myEntries = in.myEntries + shift;
  return x;
}

__device__ __forceinline__ void advanceExchangeIfLast(const RowReduceExchange &x, unsigned long long ticket, unsigned int parts) {
  if (static_cast<unsigned int>(ticket) != parts - 1u) return;
  const unsigned int step = x.epoch - static_cast<unsigned int>(ticket >> 32);  // 1, or 3 across the wrap
  atomicAdd(x.callWord, (static_cast<unsigned long long>(step) << 32) - parts);
}

// All threads of the CTA call this once, before any of them sends: thread 0 takes the CTA's ticket and leaves the
// call's view of the exchange in shared memory, where the sends and the reads of the entries pick it up.  (Kept in
// registers instead, the view's ten pointers stay live across the streaming loop, and that loop then ran 7 % slower:
// measured with the exchange itself switched off.)
__device__ __forceinline__ const RowReduceExchange &joinExchangeCall(const RowReduceExchange &in) {
  __shared__ RowReduceExchange ctaExchange;
  if (threadIdx.x == 0) {
    const unsigned long long ticket = takeExchangeTicket(in);
    ctaExchange = resolveExchange(in, ticket);
    advanceExchangeIfLast(ctaExchange, ticket, gridDim.x);
  }
  __syncthreads();
  return ctaExchange;
}

__device__ __forceinline__ void sendPartial(const RowReduceExchange &x, long long row, float v) {
  const unsigned long long entry = (static_cast<unsigned long long>(x.epoch) << 32) | __float_as_uint(v);
  for (int p = 0; p < x.world; ++p)
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(x.peerEntries[p] + row), "l"(entry) : "memory");
}

// The same by a whole warp: lane p stores to rank p, so the stores leave together (v is lane 0's).
__device__ __forceinline__ void sendPartialByWarp(const RowReduceExchange &x, long long row, float v, int lane) {
  v = __shfl_sync(0xffffffffu, v, 0);
  const unsigned long long entry = (static_cast<unsigned long long>(x.epoch) << 32) | __float_as_uint(v);
  if (lane < x.world)
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(x.peerEntries[lane] + row), "l"(entry) : "memory");
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

// One warp finishes up to 32 / world rows at once: rows first, first + step, ...; lane slot * world + p fetches
// rank p's partial sum of row `slot`, the slot's first lane adds them in rank order and stores the sum.
template <class P>
__device__ __forceinline__ bool finishRowsByWarp(const RowReduceExchange &x, void *out, long long first, long long step, int count, int lane) {
  const int slot = lane / x.world, p = lane - slot * x.world;
  const bool mine = slot < count;
  const long long row = first + slot * step;
  unsigned long long w = 0;
  bool ok = true;
  if (mine) ok = awaitEntry(x.myEntries + p * x.slotStride + row, x.epoch, w);
  ok = __all_sync(0xffffffffu, ok) != 0;
  float t = 0.f;
  for (int q = 0; q < x.world; ++q) t += __uint_as_float(__shfl_sync(0xffffffffu, static_cast<unsigned int>(w), (lane + q) & 31));
  if (ok && mine && p == 0) storeSum<P>(out, row, t);
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

template <class P, class B, bool VECTOR, bool XCHG = false>
__device__ __forceinline__ void rowReduceTeams(const RrParams &prm) {
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
  const RowReduceExchange &xr = XCHG ? joinExchangeCall(prm.xchg) : prm.xchg;

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
          if (VECTOR && B::kInterpreted) {
            if (v0 + u * L < vEnd) {  // the interpreted body decodes its ops once per 16-byte vector
              const uint4 y16 = evalVector16<B, P, NV>(raw[u], prm.prog);
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
      if (XCHG) sendPartial(xr, row, sum);
      else if (prm.slices > 1) prm.partial[row * prm.slices + slice] = sum;
      else storeSum<P>(prm.out, row, sum);
    }
  }
  if constexpr (XCHG) exchangeTail<P>(xr, prm.out, prm.rows);
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
constexpr unsigned int kStreamBytesInFlight = 64 * 1024;   // per SM: short rows deepen the ring until warps x stages x chunk reaches this
constexpr int kStreamMinRowBytes = 4096;                   // shorter rows go to the team-per-row kernel (measured: 2 KB rows
                                                           // reach 0.63 of the copy rate staged, 0.75 with plain loads)
constexpr unsigned long long kStreamWaitLimitNs = 2000000000ull;

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
  unsigned int *status;          // set to 1 when a wait for a staged copy ran out
  BodyProgram prog;
  RowReduceExchange xchg;        // world > 0: the sums are partial and go to every rank's mailbox
  int finishLag;                 // exchange: rows a warp streams on after sending one before it reads that row's entries
};

__device__ __forceinline__ unsigned int smemU32(const void *p) { return static_cast<unsigned int>(__cvta_generic_to_shared(p)); }

template <class P, class B, bool XCHG = false>
__device__ __forceinline__ void rowReduceStream(const RrStreamParams &prm, unsigned char *streamSmem) {
  constexpr int NV = B::kViews;
  constexpr int kElemBytes = sizeof(typename P::Scalar);
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
  long long pendFirst = firstRow;  // exchange: the oldest row this warp has sent but not yet finished ...
  int pending = 0;                 // ... and how many such rows there are (rows pendFirst, pendFirst + totalWarps, ...)
  const RowReduceExchange &xr = XCHG ? joinExchangeCall(prm.xchg) : prm.xchg;  // the ring's first copies are already in flight
  const int finishGroup = XCHG ? 32 / max(xr.world, 1) : 1;
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
            atomicCAS(prm.status, 0u, 1u);
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
          if constexpr (B::kInterpreted) {
            uint4 all[NV];
#pragma unroll
            for (int k = 0; k < NV; ++k)
              all[k] = k == prm.streamViewIndex ? raw : make_uint4(bcastNow[k], bcastNow[k], bcastNow[k], bcastNow[k]);
            const uint4 y16 = evalVector16<B, P, NV>(all, prm.prog);
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
      sendPartialByWarp(xr, row, sum, lane);
      ++pending;
      if (pending >= finishGroup + prm.finishLag) {  // the oldest group has had finishLag rows' time to arrive
        if (peersAnswer) peersAnswer = finishRowsByWarp<P>(xr, prm.out, pendFirst, totalWarps, finishGroup, lane);
        pendFirst += finishGroup * totalWarps;
        pending -= finishGroup;
      }
    } else {
      if (lane == 0) storeSum<P>(prm.out, row, sum);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) bcastNow[k] = bcastNext[k];
  }
  if constexpr (XCHG) {
    for (; pending > 0; pending -= finishGroup, pendFirst += finishGroup * totalWarps)
      if (peersAnswer) peersAnswer = finishRowsByWarp<P>(xr, prm.out, pendFirst, totalWarps, min(pending, finishGroup), lane);
    if (!peersAnswer && lane == 0) atomicExch(xr.status, 1u);
  }
}

template <class P>
__device__ __forceinline__ void rowReduceFinalize(const float *__restrict__ partial, void *out, long long rows, int slices) {
  const long long row = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float t = 0.f;
  for (int s = 0; s < slices; ++s) t += partial[row * slices + s];
  storeSum<P>(out, row, t);
}

} // namespace kernels
} // namespace afir
