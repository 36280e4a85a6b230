// Matmul + bias + LeakyReLU fused group for sm_100a:
//     out[M,N] = epilogue(A[M,K] . B[K,N] + bias[N]),  epilogue(x) = max(x, alpha * x)
// (semantics: lib/Conversion/MarkStructuredOps/AnnotateMixMatmulSemanticsPass.cpp:171-242 --
// BiasAdd then maximumf(x, mulf(x, alpha)); the reference runs the matmul on the cube unit and
// re-reads C from global memory for the LeakyRelu, lib/Target/CannKernel/CannTranslation.cpp:1573-1615;
// here the epilogue is applied to the accumulator before it ever leaves the SM).
//
// Structure (one persistent CTA per SM, no clusters, no multicast):
//   warp 0      TMA producer: A tile [TM x 64] (K-major, 128B swizzle) and B tile [64 x 256]
//               (N-major, four 64x64 boxes, 128B swizzle) into a ring of shared-memory stages;
//   warp 1      MMA issuer: tcgen05.mma.cta_group::1.kind::f16, 128x256x16 per instruction,
//               f32 accumulators in tensor memory (2 x 256 columns); also owns TMEM alloc/free;
//   warps 2..   epilogue: tcgen05.ld the accumulator (one row per thread), + bias, LeakyReLU,
//               convert, 16-byte stores.
// TM = 128 * MB.  MB = 1: the two TMEM accumulators double-buffer consecutive tiles (epilogue of tile
// i overlaps the mainloop of tile i+1).  MB = 2: a 256x256 tile uses both accumulators, halving the
// L2->SM operand traffic per flop (A and B are each read once per 256 rows/columns instead of 128).
//
// Every wait on an mbarrier is bounded: after ~2 s the waiting thread records a status word, raises a
// CTA-wide abort flag and every role leaves its loop; the CTA then waits (bounded) for TMA copies still
// in flight, frees its tensor memory and returns.  The host reports the status as an error.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "kernels/kernels.h"
#include "kernels/launch_util.h"
#include "kernels/matmul_plan.h"

namespace afir {
namespace kernels {
namespace {

constexpr int kBlockN = 256;
constexpr int kBlockK = 64;           // 64 x 2 bytes = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kTmemCols = 512;
constexpr int kBBoxBytes = 64 * 64 * 2;   // one 64(k) x 64(n) box
constexpr int kBStageBytes = 4 * kBBoxBytes;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// status word: 0 = ok, else (code << 8) | role.  A launch that brings its own word (the executor points it into
// its workspace, so executors sharing a device do not read each other's time-outs) uses that; otherwise this one.
__device__ unsigned int g_matmulStatus = 0;

// Per-CTA abort state in shared memory: raised by the first wait that runs out, seen by every role's next check.
struct AbortState {
  int flag;
  unsigned int *status;  // where the time-out is reported
};

struct GemmParams {
  int M, N, K;
  int numTilesM, numTilesN, numKBlocks;
  const void *bias;
  void *out;
  int biasType, epilogue;
  float alpha;
  unsigned int idesc;
  unsigned int *status;  // device word for wait time-outs, or null for the library's own
  int tileN;  // columns per CTA tile: 256, or less (a multiple of 32) when that fills the last wave of CTAs
  int band;  // tile-rows per raster band
  int bKMajor;  // 1: B is given as [N, K] (out = A x B^T, the layout of a torch Linear weight): K-major tiles like A's
};

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ unsigned int smemAddr(const void *p) {
  return static_cast<unsigned int>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbarInit(unsigned int bar, unsigned int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(unsigned int bar, unsigned int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(unsigned int bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(unsigned int bar, unsigned int parity) {
  unsigned int done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait.  Returns false when the abort flag is (or becomes) raised.
__device__ __forceinline__ bool mbarWait(unsigned int bar, unsigned int parity, volatile AbortState *abortFlag, unsigned int role) {
  if (mbarTryWait(bar, parity)) return true;
  const unsigned long long t0 = globalTimerNs();
  unsigned int spins = 0;
  while (true) {
    if (mbarTryWait(bar, parity)) return true;
    // epilogue warps wait a whole mainloop for their accumulator: back off instead of burning issue slots and power
    if (role == 2) __nanosleep(256);
    else if (role == 0) __nanosleep(64);  // the producer is normally a full ring ahead: poll lazily
    if ((++spins & 63u) == 0) {
      if (abortFlag->flag) return false;
      if (globalTimerNs() - t0 > kWaitLimitNs) {
        abortFlag->flag = 1;
        atomicCAS(abortFlag->status, 0u, (1u << 8) | role);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tmaLoad2d(unsigned int dst, const CUtensorMap *map, int x, int y, unsigned int bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tcgen05FenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05FenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmemAlloc(unsigned int dstSmem, unsigned int cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dstSmem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDealloc(unsigned int taddr, unsigned int cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void ummaF16(unsigned int dTmem, unsigned long long aDesc, unsigned long long bDesc,
                                        unsigned int idesc, unsigned int accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void ummaCommit(unsigned int bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmemLoad32(unsigned int taddr, unsigned int (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (tcgen05): start address, leading/stride byte offsets (>>4),
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ unsigned long long smemDesc(unsigned int addr, unsigned int lboBytes, unsigned int sboBytes) {
  unsigned long long d = 0;
  d |= static_cast<unsigned long long>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<unsigned long long>((lboBytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<unsigned long long>((sboBytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version (Blackwell)
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// Eight consecutive bias values as f32 (n is a multiple of 8: 16-byte aligned for 16-bit types).
__device__ __forceinline__ void loadBias8(const void *bias, int type, int n, float (&b)[8]) {
  if (type == kF32) {
    const float4 lo = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(bias) + n));
    const float4 hi = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(bias) + n) + 1);
    b[0] = lo.x; b[1] = lo.y; b[2] = lo.z; b[3] = lo.w; b[4] = hi.x; b[5] = hi.y; b[6] = hi.z; b[7] = hi.w;
    return;
  }
  const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(bias) + n));
  const unsigned int w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (type == kF16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      b[2 * i] = f.x;
      b[2 * i + 1] = f.y;
    } else {
      b[2 * i] = __uint_as_float(w[i] << 16);
      b[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
}

// Eight f32 results -> 16-byte pieces of the output row (two pieces for f32, one for 16-bit types).
template <int OUT> struct OutPack;
template <> struct OutPack<kF32> {
  static constexpr int kBytes = 4;
  static constexpr int kPieces = 2;
  __device__ __forceinline__ static void pack8(const float *v, uint4 *q) {
    q[0] = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    q[1] = make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7]));
  }
};
template <> struct OutPack<kBF16> {
  static constexpr int kBytes = 2;
  static constexpr int kPieces = 1;
  __device__ __forceinline__ static void pack8(const float *v, uint4 *q) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    q[0] = make_uint4(*reinterpret_cast<unsigned int *>(&a), *reinterpret_cast<unsigned int *>(&b),
                      *reinterpret_cast<unsigned int *>(&c), *reinterpret_cast<unsigned int *>(&d));
  }
};
template <> struct OutPack<kF16> {
  static constexpr int kBytes = 2;
  static constexpr int kPieces = 1;
  __device__ __forceinline__ static void pack8(const float *v, uint4 *q) {
    __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
    q[0] = make_uint4(*reinterpret_cast<unsigned int *>(&a), *reinterpret_cast<unsigned int *>(&b),
                      *reinterpret_cast<unsigned int *>(&c), *reinterpret_cast<unsigned int *>(&d));
  }
};

// shared-memory control block (after the operand ring)
template <int STAGES> struct Control {
  unsigned long long full[STAGES];
  unsigned long long empty[STAGES];
  unsigned long long tmemFull[2];
  unsigned long long tmemEmpty[2];
  unsigned int tmemBase;
  AbortState abortFlag;
};

template <int MB> struct Shape {
  static constexpr int kTileM = 128 * MB;
  static constexpr int kAStageBytes = kTileM * kBlockK * 2;
  static constexpr int kStageBytes = kAStageBytes + kBStageBytes;
  static constexpr int kStages = MB == 1 ? 4 : 3;
  static constexpr int kEpilogueWarps = 4 * MB;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
  static constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;  // per warp: 32 rows x 128 bytes
  static constexpr size_t kSmemBytes =
      1024 + static_cast<size_t>(kStages) * kStageBytes + kStagingBytes + sizeof(Control<kStages>);
};

// One accumulator tile of one epilogue warp: wait for the accumulator, + bias, activation, convert,
// write 32 rows x 256 columns.  `arriveEmpty` (called by lane 0) hands the accumulator back to the MMA
// warp.  Returns false when the bounded wait gave up.
template <int OUT, class ArriveEmpty>
__device__ __forceinline__ bool epilogueTile(const GemmParams &prm, unsigned char *stg, unsigned int taddr, int rowBase, int tn,
                                             int lane, unsigned int fullBar, unsigned int fullParity,
                                             volatile AbortState *abortFlag, ArriveEmpty arriveEmpty) {
      constexpr int kColsPerSlice = 128 / OutPack<OUT>::kBytes;  // 64 (16-bit) or 32 (f32)

      // Writes one 128-byte slice per row (parked in `stg`, 16-byte pieces XOR-swizzled by row so both
      // phases are bank-conflict free) with 8 lanes per row: every warp store covers four full
      // 128-byte lines of the output instead of 32 scattered 16-byte pieces.
      auto storeSlice = [&](int c) {
        __syncwarp();
        const int piece = lane & 7;
        const int colInTile = c + piece * (16 / OutPack<OUT>::kBytes);
        const int ncol = tn * prm.tileN + colInTile;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3);
          const uint4 val = *reinterpret_cast<const uint4 *>(stg + rr * 128 + ((piece ^ (rr & 7)) << 4));
          const int grow = rowBase + rr;
          if (grow < prm.M && ncol < prm.N && colInTile < prm.tileN)  // N and tileN are multiples of 8: a 16-byte piece is wholly inside or outside
            *reinterpret_cast<uint4 *>(static_cast<unsigned char *>(prm.out) +
                                       (static_cast<size_t>(grow) * prm.N + ncol) * OutPack<OUT>::kBytes) = val;
        }
        __syncwarp();
      };
      auto activate = [&](float x) {
        if (prm.epilogue == kEpiBiasAddLeakyRelu) return fmaxf(x, x * prm.alpha);
        if (prm.epilogue == kEpiBiasAddRelu) return fmaxf(x, 0.0f);
        return x;
      };

      if constexpr (OutPack<OUT>::kBytes == 2) {
        // 16-bit outputs: the whole row (256 columns) fits in registers once converted, so the
        // accumulator is drained first and tensor memory handed back to the MMA warp before any
        // global store is issued; the stores then overlap the next tile's mainloop.
        // Bias of the tile's 256 columns, as f32, sits in this warp's staging area during the drain
        // (the area is idle until the store phase); it is fetched before waiting for the accumulator.
        float *biasS = reinterpret_cast<float *>(stg);
        if (prm.epilogue != kEpiNone) {
          const int n = tn * prm.tileN + lane * 8;
          float bv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (n < prm.N) loadBias8(prm.bias, prm.biasType, n, bv);
          reinterpret_cast<float4 *>(biasS + lane * 8)[0] = make_float4(bv[0], bv[1], bv[2], bv[3]);
          reinterpret_cast<float4 *>(biasS + lane * 8)[1] = make_float4(bv[4], bv[5], bv[6], bv[7]);
        }
        __syncwarp();
        if (!mbarWait(fullBar, fullParity, abortFlag, 2)) return false;
        tcgen05FenceAfter();
        uint4 packed[kBlockN / 8];
#pragma unroll
        for (int cc = 0; cc < kBlockN / 32; ++cc) {
          if (cc * 32 >= prm.tileN) {  // a narrower tile: these accumulator columns were not written
#pragma unroll
            for (int j = 0; j < 4; ++j) packed[cc * 4 + j] = make_uint4(0u, 0u, 0u, 0u);
            continue;
          }
          unsigned int r[32];
          tmemLoad32(taddr + cc * 32, r);
          tmemLoadWait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
            if (prm.epilogue != kEpiNone) {
              b0 = *reinterpret_cast<const float4 *>(biasS + cc * 32 + j * 8);
              b1 = *reinterpret_cast<const float4 *>(biasS + cc * 32 + j * 8 + 4);
            }
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = activate(__uint_as_float(r[j * 8 + e]) + bv[e]);
            OutPack<OUT>::pack8(v, &packed[cc * 4 + j]);
          }
        }
        tcgen05FenceBefore();
        __syncwarp();
        if (lane == 0) arriveEmpty();
#pragma unroll
        for (int sl = 0; sl < kBlockN / kColsPerSlice; ++sl) {
          if (sl * kColsPerSlice >= prm.tileN) continue;
#pragma unroll
          for (int piece = 0; piece < 8; ++piece)
            *reinterpret_cast<uint4 *>(stg + lane * 128 + ((piece ^ (lane & 7)) << 4)) = packed[sl * 8 + piece];
          storeSlice(sl * kColsPerSlice);
        }
      } else {
        // f32 outputs: a row does not fit in registers; convert and store slice by slice, then release.
        if (!mbarWait(fullBar, fullParity, abortFlag, 2)) return false;
        tcgen05FenceAfter();
#pragma unroll 1
        for (int c = 0; c < prm.tileN; c += kColsPerSlice) {
          unsigned int r[32];
          tmemLoad32(taddr + c, r);
          tmemLoadWait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = tn * prm.tileN + c + j * 8;
            float bv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (prm.epilogue != kEpiNone && n < prm.N) loadBias8(prm.bias, prm.biasType, n, bv);
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = activate(__uint_as_float(r[j * 8 + e]) + bv[e]);
            uint4 q[OutPack<OUT>::kPieces];
            OutPack<OUT>::pack8(v, q);
#pragma unroll
            for (int pce = 0; pce < OutPack<OUT>::kPieces; ++pce) {
              const int piece = j * OutPack<OUT>::kPieces + pce;
              *reinterpret_cast<uint4 *>(stg + lane * 128 + ((piece ^ (lane & 7)) << 4)) = q[pce];
            }
          }
          storeSlice(c);
        }
        tcgen05FenceBefore();
        __syncwarp();
        if (lane == 0) arriveEmpty();
      }
  return true;
}

template <int MB, int OUT>
__global__ void __launch_bounds__(Shape<MB>::kThreads, 1)
matmulBiasActKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                    const __grid_constant__ GemmParams prm) {
  using S = Shape<MB>;
  constexpr int STAGES = S::kStages;
  extern __shared__ unsigned char smemRaw[];
  // 128-byte-swizzled tiles want 1024-byte alignment
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  unsigned char *staging = smem + static_cast<size_t>(STAGES) * S::kStageBytes;
  Control<STAGES> *ctl = reinterpret_cast<Control<STAGES> *>(staging + S::kStagingBytes);
  volatile AbortState *abortFlag = &ctl->abortFlag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int numTiles = prm.numTilesM * prm.numTilesN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbarInit(smemAddr(&ctl->full[s]), 1);
      mbarInit(smemAddr(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&ctl->tmemFull[a]), 1);
      mbarInit(smemAddr(&ctl->tmemEmpty[a]), MB == 1 ? 4 : 4);  // one arrival per epilogue warp of that accumulator
    }
    ctl->abortFlag.flag = 0;
    ctl->abortFlag.status = prm.status ? prm.status : &g_matmulStatus;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetchTensorMap(&mapA);
    prefetchTensorMap(&mapB);
  }
  if (warp == 1) {
    tmemAlloc(smemAddr(&ctl->tmemBase), kTmemCols);
    tmemRelinquish();
  }
  tcgen05FenceBefore();
  __syncthreads();
  tcgen05FenceAfter();
  const unsigned int tmemBase = ctl->tmemBase;

  // Tile order: M fastest inside bands of 16 tile-rows so that concurrently running CTAs share
  // A row-panels and B column-panels in L2.
  auto tileCoords = [&](int t, int &tm, int &tn) {
    const int kBand = prm.band;
    const int bandTiles = kBand * prm.numTilesN;
    const int band = t / bandTiles;
    const int within = t - band * bandTiles;
    const int rowsInBand = min(kBand, prm.numTilesM - band * kBand);
    tm = band * kBand + within % rowsInBand;
    tn = within / rowsInBand;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      unsigned int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
        int tm, tn;
        tileCoords(t, tm, tn);
        for (int kb = 0; kb < prm.numKBlocks; ++kb, ++it) {
          const int s = it % STAGES;
          const unsigned int phase = (it / STAGES) & 1u;
          if (!mbarWait(smemAddr(&ctl->empty[s]), phase ^ 1u, abortFlag, 0)) { ok = false; break; }
          const unsigned int full = smemAddr(&ctl->full[s]);
          mbarExpectTx(full, S::kStageBytes);
          unsigned char *stage = smem + static_cast<size_t>(s) * S::kStageBytes;
          tmaLoad2d(smemAddr(stage), &mapA, kb * kBlockK, tm * S::kTileM, full);
          if (prm.bKMajor) {  // one [256 n-rows x 64 k] box, the same bytes as the four N-major boxes
            tmaLoad2d(smemAddr(stage + S::kAStageBytes), &mapB, kb * kBlockK, tn * prm.tileN, full);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tmaLoad2d(smemAddr(stage + S::kAStageBytes + j * kBBoxBytes), &mapB, tn * prm.tileN + j * 64, kb * kBlockK, full);
          }
        }
      }
      if (!ok) {
        // loads already issued still land in this CTA's shared memory: give them time before leaving
        for (int s = 0; s < STAGES; ++s) {
          const unsigned long long t0 = globalTimerNs();
          while (!mbarTryWait(smemAddr(&ctl->full[s]), 0) && !mbarTryWait(smemAddr(&ctl->full[s]), 1) &&
                 globalTimerNs() - t0 < 1000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      unsigned int it = 0, tileIter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileIter) {
        // accumulator(s) of this tile and the parity of their "drained" barrier
        const int acc0 = MB == 1 ? static_cast<int>(tileIter & 1u) : 0;
        const unsigned int use = MB == 1 ? (tileIter >> 1) : tileIter;  // how many times this accumulator was used before
        for (int h = 0; h < MB && ok; ++h)
          if (!mbarWait(smemAddr(&ctl->tmemEmpty[acc0 + h]), (use & 1u) ^ 1u, abortFlag, 1)) ok = false;
        if (!ok) break;
        tcgen05FenceAfter();
        for (int kb = 0; kb < prm.numKBlocks; ++kb, ++it) {
          const int s = it % STAGES;
          const unsigned int phase = (it / STAGES) & 1u;
          if (!mbarWait(smemAddr(&ctl->full[s]), phase, abortFlag, 1)) { ok = false; break; }
          tcgen05FenceAfter();
          const unsigned int aBase = smemAddr(smem + static_cast<size_t>(s) * S::kStageBytes);
          const unsigned int bBase = aBase + S::kAStageBytes;
#pragma unroll
          for (int h = 0; h < MB; ++h) {
            const unsigned int dTmem = tmemBase + static_cast<unsigned int>((acc0 + h) * kBlockN);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              // A: K-major, rows 128 B apart, 8-row groups 1024 B apart; 16 k-elements = 32 bytes along the row
              const unsigned long long aDesc = smemDesc(aBase + h * (128 * kBlockK * 2) + k * (kUmmaK * 2), 16, 1024);
              // B: N-major, 64-column blocks 8192 B apart (leading), 8-row k-groups 1024 B apart (stride);
              // 16 k-rows = two k-groups = 2048 bytes
              // (given as [N, K]: K-major like A, n-rows 128 B apart, 8-row groups 1024 B apart, 32 bytes per k-step)
              const unsigned long long bDesc = prm.bKMajor ? smemDesc(bBase + k * (kUmmaK * 2), 16, 1024)
                                                           : smemDesc(bBase + k * (kUmmaK * 128), kBBoxBytes, 1024);
              ummaF16(dTmem, aDesc, bDesc, prm.idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          ummaCommit(smemAddr(&ctl->empty[s]));  // frees the stage when these MMAs have read it
        }
        if (!ok) break;
        for (int h = 0; h < MB; ++h) ummaCommit(smemAddr(&ctl->tmemFull[acc0 + h]));
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int ew = warp - 2;                 // 0 .. 4*MB-1
    const int half = ew / 4;                 // which accumulator of an MB=2 tile
    const int quarter = warp & 3;            // TMEM lanes this warp may touch: [32*quarter, 32*quarter+32)
    unsigned int tileIter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileIter) {
      int tm, tn;
      tileCoords(t, tm, tn);
      const int acc = MB == 1 ? static_cast<int>(tileIter & 1u) : half;
      const unsigned int use = MB == 1 ? (tileIter >> 1) : tileIter;
      const int rowBase = tm * S::kTileM + half * 128 + quarter * 32;
      const unsigned int taddr = tmemBase + static_cast<unsigned int>(acc * kBlockN) + (static_cast<unsigned int>(quarter * 32) << 16);
      const unsigned int emptyBar = smemAddr(&ctl->tmemEmpty[acc]);
      if (!epilogueTile<OUT>(prm, staging + ew * (32 * 128), taddr, rowBase, tn, lane, smemAddr(&ctl->tmemFull[acc]), use & 1u,
                             abortFlag, [&] { mbarArrive(emptyBar); })) {
        ok = false;
        break;
      }
    }
  }

  // ---------------- teardown ----------------
  tcgen05FenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcgen05FenceAfter();
    tmemDealloc(tmemBase, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------------
// Two-CTA variant (tcgen05 cta_group::2): a cluster of two CTAs on neighbouring SMs computes one
// 256x256 tile.  CTA r holds A rows [128r, 128r+128) and B columns [128r, 128r+128) of the tile in its own
// shared memory and the accumulator rows [128r, 128r+128) x 256 columns in its own tensor memory; the
// leader CTA (rank 0) issues one 256x256x16 instruction for the pair.  Per SM and k-block this moves
// 32 KB into shared memory and reads 8 KB per instruction out of it, half of what the single-CTA kernel
// needs, which is what shared-memory bandwidth allows at full tensor rate; the accumulator takes 256 of
// the 512 tensor-memory columns, so two tiles are double-buffered and the epilogue overlaps the mainloop.
// No multicast anywhere: every CTA loads its own operand halves; the peer's loads complete on the
// leader's "full" barrier, the leader's commits arrive on both CTAs' "empty"/"accumulator full"
// barriers (one commit each), the peer's epilogue warps arrive remotely on the leader's
// "accumulator drained" barrier.  All waits are bounded as in the single-CTA kernel.
// ---------------------------------------------------------------------------------------------------
constexpr int k2Stages = 6;
constexpr int k2AStageBytes = 128 * kBlockK * 2;
constexpr int k2BStageBytes = 2 * kBBoxBytes;
constexpr int k2StageBytes = k2AStageBytes + k2BStageBytes;
constexpr int k2Threads = 192;
constexpr int k2StagingBytes = 4 * 32 * 128;
constexpr size_t k2SmemBytes = 1024 + static_cast<size_t>(k2Stages) * k2StageBytes + k2StagingBytes + sizeof(Control<k2Stages>);

__device__ __forceinline__ unsigned int clusterCtaRank() {
  unsigned int r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ unsigned int mapToCta(unsigned int addr, unsigned int rank) {
  unsigned int r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void clusterSyncAll() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbarArriveRemote(unsigned int clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
__device__ __forceinline__ void tmaLoad2dPair(unsigned int dst, const CUtensorMap *map, int x, int y, unsigned int clusterBar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(clusterBar)
      : "memory");
}
__device__ __forceinline__ void ummaF16Pair(unsigned int dTmem, unsigned long long aDesc, unsigned long long bDesc,
                                            unsigned int idesc, unsigned int accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void ummaCommitPair(unsigned int clusterBar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(clusterBar) : "memory");
}

template <int OUT>
__global__ void __launch_bounds__(k2Threads, 1)
matmulBiasActPairKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                        const __grid_constant__ GemmParams prm) {
  extern __shared__ unsigned char smemRaw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  unsigned char *staging = smem + static_cast<size_t>(k2Stages) * k2StageBytes;
  Control<k2Stages> *ctl = reinterpret_cast<Control<k2Stages> *>(staging + k2StagingBytes);
  volatile AbortState *abortFlag = &ctl->abortFlag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const unsigned int rank = clusterCtaRank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int numPairs = gridDim.x >> 1;
  const int numTiles = prm.numTilesM * prm.numTilesN;  // 256 x 256 tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      mbarInit(smemAddr(&ctl->full[s]), 1);   // leader: its own arrive.expect_tx covers both CTAs' bytes
      mbarInit(smemAddr(&ctl->empty[s]), 1);  // one commit from the leader
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&ctl->tmemFull[a]), 1);
      mbarInit(smemAddr(&ctl->tmemEmpty[a]), 8);  // four epilogue warps in each CTA (leader's copy is the one used)
    }
    ctl->abortFlag.flag = 0;
    ctl->abortFlag.status = prm.status ? prm.status : &g_matmulStatus;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetchTensorMap(&mapA);
    prefetchTensorMap(&mapB);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&ctl->tmemBase)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05FenceBefore();
  __syncthreads();
  clusterSyncAll();  // both CTAs' barriers exist before anyone signals across
  tcgen05FenceAfter();
  const unsigned int tmemBase = ctl->tmemBase;

  auto tileCoords = [&](int t, int &tm, int &tn) {
    const int kBand = prm.band;
    const int bandTiles = kBand * prm.numTilesN;
    const int band = t / bandTiles;
    const int within = t - band * bandTiles;
    const int rowsInBand = min(kBand, prm.numTilesM - band * kBand);
    tm = band * kBand + within % rowsInBand;
    tn = within / rowsInBand;
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      unsigned int it = 0;
      bool ok = true;
      for (int t = pair; t < numTiles && ok; t += numPairs) {
        int tm, tn;
        tileCoords(t, tm, tn);
        for (int kb = 0; kb < prm.numKBlocks; ++kb, ++it) {
          const int s = it % k2Stages;
          const unsigned int phase = (it / k2Stages) & 1u;
          if (!mbarWait(smemAddr(&ctl->empty[s]), phase ^ 1u, abortFlag, 0)) { ok = false; break; }
          const unsigned int fullLocal = smemAddr(&ctl->full[s]);
          if (rank == 0) mbarExpectTx(fullLocal, 2 * k2StageBytes);
          const unsigned int fullLeader = mapToCta(fullLocal, 0);
          unsigned char *stage = smem + static_cast<size_t>(s) * k2StageBytes;
          tmaLoad2dPair(smemAddr(stage), &mapA, kb * kBlockK, tm * 256 + static_cast<int>(rank) * 128, fullLeader);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tmaLoad2dPair(smemAddr(stage + k2AStageBytes + j * kBBoxBytes), &mapB,
                          tn * kBlockN + static_cast<int>(rank) * 128 + j * 64, kb * kBlockK, fullLeader);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (lane == 0 && rank == 0) {
      unsigned int it = 0, tileIter = 0;
      bool ok = true;
      for (int t = pair; t < numTiles && ok; t += numPairs, ++tileIter) {
        const int acc = static_cast<int>(tileIter & 1u);
        const unsigned int use = tileIter >> 1;
        if (!mbarWait(smemAddr(&ctl->tmemEmpty[acc]), (use & 1u) ^ 1u, abortFlag, 1)) break;
        tcgen05FenceAfter();
        const unsigned int dTmem = tmemBase + static_cast<unsigned int>(acc * kBlockN);
        for (int kb = 0; kb < prm.numKBlocks; ++kb, ++it) {
          const int s = it % k2Stages;
          const unsigned int phase = (it / k2Stages) & 1u;
          if (!mbarWait(smemAddr(&ctl->full[s]), phase, abortFlag, 1)) { ok = false; break; }
          tcgen05FenceAfter();
          const unsigned int aBase = smemAddr(smem + static_cast<size_t>(s) * k2StageBytes);
          const unsigned int bBase = aBase + k2AStageBytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const unsigned long long aDesc = smemDesc(aBase + k * (kUmmaK * 2), 16, 1024);
            const unsigned long long bDesc = smemDesc(bBase + k * (kUmmaK * 128), kBBoxBytes, 1024);
            ummaF16Pair(dTmem, aDesc, bDesc, prm.idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          const unsigned int emptyLocal = smemAddr(&ctl->empty[s]);
          ummaCommitPair(emptyLocal);               // frees the stage in this CTA ...
          ummaCommitPair(mapToCta(emptyLocal, 1));  // ... and in the peer
        }
        if (!ok) break;
        const unsigned int fullAcc = smemAddr(&ctl->tmemFull[acc]);
        ummaCommitPair(fullAcc);
        ummaCommitPair(mapToCta(fullAcc, 1));
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows) ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;
    unsigned int tileIter = 0;
    for (int t = pair; t < numTiles; t += numPairs, ++tileIter) {
      int tm, tn;
      tileCoords(t, tm, tn);
      const int acc = static_cast<int>(tileIter & 1u);
      const unsigned int use = tileIter >> 1;
      const int rowBase = tm * 256 + static_cast<int>(rank) * 128 + quarter * 32;
      const unsigned int taddr = tmemBase + static_cast<unsigned int>(acc * kBlockN) + (static_cast<unsigned int>(quarter * 32) << 16);
      const unsigned int emptyLeader = mapToCta(smemAddr(&ctl->tmemEmpty[acc]), 0);
      if (!epilogueTile<OUT>(prm, staging + ew * (32 * 128), taddr, rowBase, tn, lane, smemAddr(&ctl->tmemFull[acc]), use & 1u,
                             abortFlag, [&] { mbarArriveRemote(emptyLeader); }))
        break;
    }
  }

  // ---------------- teardown ----------------
  tcgen05FenceBefore();
  __syncthreads();
  clusterSyncAll();  // the peer must not free tensor memory the leader's instructions may still write
  if (warp == 1) {
    tcgen05FenceAfter();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

bool makeMap2d(CUtensorMap *map, CUtensorMapDataType type, const void *base, uint64_t inner, uint64_t outer,
               uint64_t rowBytes, uint32_t boxInner, uint32_t boxOuter) {
  EncodeTiledFn fn = encodeTiled();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {rowBytes};
  cuuint32_t box[2] = {boxInner, boxOuter};
  cuuint32_t elemStrides[2] = {1, 1};
  return fn(map, type, 2, const_cast<void *>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A function attribute belongs to the function ON THE CURRENT DEVICE: a process that runs the matmul on several
// GPUs has to set it once on each of them.  `run` calls `set` the first time it is reached with a given device
// current (and again after a failure) and returns that device's result.
struct PerDeviceOnce {
  std::mutex mu;
  bool done[64] = {false};
  template <class F> cudaError_t run(F set) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return set();
    std::lock_guard<std::mutex> lock(mu);
    if (done[device]) return cudaSuccess;
    e = set();
    done[device] = e == cudaSuccess;
    return e;
  }
};

void fail(char *errorText, const char *msg) {
  if (errorText) std::snprintf(errorText, 256, "%s", msg);
}

template <int MB, int OUT>
int launchVariant(const CUtensorMap &mapA, const CUtensorMap &mapB, const GemmParams &p, int grid, cudaStream_t stream,
                  char *errorText) {
  using S = Shape<MB>;
  auto kernel = matmulBiasActKernel<MB, OUT>;
  static PerDeviceOnce reserved;
  const cudaError_t attrErr = reserved.run([&] {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S::kSmemBytes));
  });
  if (attrErr != cudaSuccess) {
    fail(errorText, "matmul: cannot reserve shared memory for the operand ring");
    return static_cast<int>(attrErr);
  }
  launchOrdinary(kernel, grid, S::kThreads, S::kSmemBytes, stream, mapA, mapB, p);
  return static_cast<int>(cudaGetLastError());
}

template <int OUT>
int launchPairVariant(const CUtensorMap &mapA, const CUtensorMap &mapB, const GemmParams &p, int grid, cudaStream_t stream,
                      char *errorText) {
  auto kernel = matmulBiasActPairKernel<OUT>;
  static PerDeviceOnce reserved;
  const cudaError_t attrErr = reserved.run([&] {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(k2SmemBytes));
  });
  if (attrErr != cudaSuccess) {
    fail(errorText, "matmul: cannot reserve shared memory for the operand ring");
    return static_cast<int>(attrErr);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned int>(grid), 1, 1);
  cfg.blockDim = dim3(k2Threads, 1, 1);
  cfg.dynamicSmemBytes = k2SmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, mapA, mapB, p));
}

} // namespace

int launchMatmul(const MatmulLaunch &l, cudaStream_t stream, int *launched, char *errorText) {
  if (launched) *launched = 0;
  if (l.M == 0 || l.N == 0) return 0;
  if (l.inType != kF16 && l.inType != kBF16) { fail(errorText, "matmul: A and B must be f16 or bf16"); return 1; }
  if (l.K <= 0) { fail(errorText, "matmul: K must be positive"); return 1; }
  if (l.K % 8 != 0 || l.N % 8 != 0) {
    fail(errorText, "matmul: K and N must be multiples of 8 (16-byte rows for the TMA tensor maps)");
    return 1;
  }
  if ((reinterpret_cast<uintptr_t>(l.A) | reinterpret_cast<uintptr_t>(l.B) | reinterpret_cast<uintptr_t>(l.out)) & 15u) {
    fail(errorText, "matmul: A, B and out must be 16-byte aligned");
    return 1;
  }
  if (l.M >= (1ll << 31) || l.N >= (1ll << 31) || l.K >= (1ll << 31)) { fail(errorText, "matmul: dimension too large"); return 1; }
  if (l.epilogue != kEpiNone && !l.bias) { fail(errorText, "matmul: the epilogue needs a bias vector"); return 1; }

  int device = 0;
  cudaGetDevice(&device);
  const int sms = deviceSmCount(device);
  // The plan (variant, grid, band) comes from the host planner; what follows launches exactly that.
  // l.stages forces a variant: 1 = 128-row single CTA, 2 = 256-row single CTA, 3 = CTA pair.
  MatmulProblem problem;
  problem.M = l.M; problem.N = l.N; problem.K = l.K;
  problem.transposeB = l.bTransposed != 0;
  MatmulHints hints;
  hints.variant = (l.stages >= 1 && l.stages <= 3) ? l.stages : 0;
  hints.blockDim = l.gridBlocks > 0 ? l.gridBlocks : 0;
  if (const char *e = std::getenv("AFIR_GEMM_BAND")) hints.band = std::max(1, std::atoi(e));
  if (const char *e = std::getenv("AFIR_GEMM_TILE_N")) hints.tileN = std::atoi(e);  // tuning: force the tile width
  MatmulPlan plan;
  const std::string refused = buildMatmulPlan(problem, hints, sms, plan);
  if (!refused.empty()) { fail(errorText, refused.c_str()); return 1; }
  if (l.planOut) *l.planOut = plan;
  const bool pairKernel = plan.variant == MatmulVariant::CtaPair;
  const int mb = plan.variant == MatmulVariant::Rows256 ? 2 : 1;
  const int tileM = 128 * mb;  // rows per TMA box of A (the pair kernel loads 128 rows per CTA)
  const CUtensorMapDataType dt = l.inType == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap mapA, mapB;
  if (!makeMap2d(&mapA, dt, l.A, static_cast<uint64_t>(l.K), static_cast<uint64_t>(l.M), static_cast<uint64_t>(l.K) * 2, kBlockK,
                 static_cast<uint32_t>(tileM)) ||
      !(l.bTransposed ? makeMap2d(&mapB, dt, l.B, static_cast<uint64_t>(l.K), static_cast<uint64_t>(l.N), static_cast<uint64_t>(l.K) * 2,
                                  kBlockK, kBlockN)
                      : makeMap2d(&mapB, dt, l.B, static_cast<uint64_t>(l.N), static_cast<uint64_t>(l.K), static_cast<uint64_t>(l.N) * 2, 64,
                                  kBlockK))) {
    fail(errorText, "matmul: cuTensorMapEncodeTiled failed (driver entry point missing or bad operand layout)");
    return 1;
  }

  GemmParams p = {};
  p.M = static_cast<int>(l.M);
  p.N = static_cast<int>(l.N);
  p.K = static_cast<int>(l.K);
  const int ctaTileM = pairKernel ? 256 : tileM;
  p.numTilesM = static_cast<int>((l.M + ctaTileM - 1) / ctaTileM);
  p.tileN = pairKernel ? kBlockN : plan.tileN;
  p.numTilesN = static_cast<int>((l.N + p.tileN - 1) / p.tileN);
  p.numKBlocks = static_cast<int>((l.K + kBlockK - 1) / kBlockK);
  p.bias = l.bias;
  p.out = l.out;
  p.biasType = l.biasType;
  p.epilogue = l.epilogue;
  p.alpha = l.alpha;
  p.band = plan.band;
  p.status = l.status;
  const unsigned int fmt = l.inType == kF16 ? 0u : 1u;
  // instruction descriptor: D=f32, A/B format, A K-major, B N-major, N = the tile's columns, M=128 (256 across a CTA pair)
  const unsigned int instrM = pairKernel ? 256u : 128u;
  p.bKMajor = l.bTransposed ? 1 : 0;
  const unsigned int bMajor = l.bTransposed ? 0u : 1u;  // bit 16: 0 = B K-major, 1 = B N-major
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | (bMajor << 16) | ((static_cast<unsigned int>(p.tileN) >> 3) << 17) | ((instrM >> 4) << 24);

  const int grid = static_cast<int>(plan.blockDim);

  int rc;
  if (pairKernel) {
    rc = l.outType == kF32 ? launchPairVariant<kF32>(mapA, mapB, p, grid, stream, errorText)
         : l.outType == kF16 ? launchPairVariant<kF16>(mapA, mapB, p, grid, stream, errorText)
                             : launchPairVariant<kBF16>(mapA, mapB, p, grid, stream, errorText);
  } else if (mb == 1) {
    rc = l.outType == kF32 ? launchVariant<1, kF32>(mapA, mapB, p, grid, stream, errorText)
         : l.outType == kF16 ? launchVariant<1, kF16>(mapA, mapB, p, grid, stream, errorText)
                             : launchVariant<1, kBF16>(mapA, mapB, p, grid, stream, errorText);
  } else {
    rc = l.outType == kF32 ? launchVariant<2, kF32>(mapA, mapB, p, grid, stream, errorText)
         : l.outType == kF16 ? launchVariant<2, kF16>(mapA, mapB, p, grid, stream, errorText)
                             : launchVariant<2, kBF16>(mapA, mapB, p, grid, stream, errorText);
  }
  if (rc == 0 && launched) *launched = 1;
  return rc;
}

int matmulCheckStatus(int device, char *errorText) {
  (void)device;
  unsigned int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_matmulStatus, sizeof(status)) != cudaSuccess) return 0;
  if (status == 0) return 0;
  const unsigned int zero = 0;
  cudaMemcpyToSymbol(g_matmulStatus, &zero, sizeof(zero));
  static const char *roles[] = {"TMA producer", "MMA issuer", "epilogue"};
  if (errorText)
    std::snprintf(errorText, 256, "matmul: %s gave up waiting on a pipeline barrier after 2 s (status 0x%x)",
                  roles[std::min(2u, status & 0xffu)], status);
  return 1;
}

} // namespace kernels
} // namespace afir
