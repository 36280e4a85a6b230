// 2-D transpose of 16-bit elements with the copy engine on both sides: out[c, r] = in[r, c].
//
// The register-block kernel (transpose.cu) stops at 0.93-0.94 of the copy rate whatever the shape, even when one
// side of it is a plain contiguous stream: each CTA loads, waits, permutes, stores and ends, so an SM's memory
// pipeline is refilled once per CTA generation.  Here three persistent CTAs per SM each keep a ring of 64 x 64 tiles
// in flight:
//   * a producer thread loads tiles with cp.async.bulk.tensor.2d into a ring of 128-byte-swizzled 8 KB stages
//     (mbarrier expect_tx / complete_tx; no multicast, no cluster);
//   * four warps transpose: ldmatrix.x4.trans reads four 8 x 8 blocks of a stage and hands every lane the
//     fragment of their transposes, stmatrix.x4 writes those fragments as rows of the output tile into the warp's
//     own staging buffer (also 128-byte swizzled, so both sides are bank-conflict free); warp w owns output rows
//     16w .. 16w + 15 of the tile, so the warps never wait for one another;
//   * the warp's lane 0 writes its 16 x 64 piece with cp.async.bulk.tensor.2d (global <- shared, bulk group) and goes on;
//     two staging buffers per warp, reused when the store before last has read its buffer.
// Ragged edges need no code: a load past the end of the matrix fills the stage with zeros, a store past the end is
// clipped.  Operands must be 16-byte aligned with row strides that are multiples of 16 bytes (what a tensor map
// can describe); anything else stays on the other kernels.  Every wait is bounded: after 2 s the status word is
// set, every role leaves its loop, the producer gives the loads already issued time to land, and the kernel ends.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <mutex>

#include "kernels/grid_dependency.cuh"
#include "kernels/kernels.h"
#include "kernels/launch_util.h"

namespace afir {
namespace kernels {
namespace {

constexpr int kTile = 64;                      // elements per tile edge: 64 x 2 bytes = one 128-byte swizzle row
constexpr int kTileBytes = kTile * kTile * 2;  // 8 KB
constexpr int kStages = 6;                     // 48 KB of loads in flight per CTA
constexpr int kCtasPerSm = 3;                  // 144 KB per SM, and three tiles being transposed at a time (a warp's chain per tile is latency)
constexpr int kWarps = 4;                      // transposing warps; one more warp produces
constexpr int kRowsPerWarp = kTile / kWarps;   // 16 output rows of a tile per warp
constexpr int kOutBytes = kRowsPerWarp * 128;  // 2 KB
constexpr int kOutBuffers = 2;
constexpr int kThreads = 32 * (kWarps + 1);
constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kTileBytes + kWarps * kOutBuffers * kOutBytes + 2 * kStages * 8 + 16;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// wait time-outs of launches that bring no status word of their own
__device__ unsigned int g_transposeStatus = 0;

constexpr unsigned int kSuper = 8;  // tiles are walked in squares of 8 x 8 (512 x 512 elements): see tileOf()

struct TtParams {
  unsigned int tilesX;  // tiles along the input columns
  unsigned int tilesY;  // tiles along the input rows
  int outRows;          // rows of the output = columns of the input
  unsigned long long numTiles;
  unsigned int *status;
};

__device__ __forceinline__ unsigned int smemAddr(const void *p) { return static_cast<unsigned int>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned long long globalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbarTryWait(unsigned int bar, unsigned int parity) {
  unsigned int done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait; false when it ran out or another role already gave up.
__device__ __forceinline__ bool mbarWait(unsigned int bar, unsigned int parity, volatile int *abortFlag, unsigned int *status) {
  if (mbarTryWait(bar, parity)) return true;
  const unsigned long long t0 = globalTimerNs();
  unsigned int spins = 0;
  while (true) {
    if (mbarTryWait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abortFlag) return false;
      if (globalTimerNs() - t0 > kWaitLimitNs) {
        *abortFlag = 1;
        atomicCAS(status, 0u, 1u);
        return false;
      }
    }
  }
}

// Tile t of the walk: squares of kSuper x kSuper tiles, so that the tiles in flight at one time are neighbours along
// the input rows AND along the output rows: both the loads and the stores of a moment then fall into runs of
// kSuper x 128 bytes per row instead of lone 128-byte pieces, each in a DRAM page of its own.  False for the tiles of
// a border square that lie outside the matrix.
__device__ __forceinline__ bool tileOf(const TtParams &p, unsigned long long t, int &tx, int &ty) {
  const unsigned int supersX = (p.tilesX + kSuper - 1) / kSuper;
  const unsigned long long st = t / (kSuper * kSuper);
  const unsigned int within = static_cast<unsigned int>(t % (kSuper * kSuper));
  tx = static_cast<int>(static_cast<unsigned int>(st % supersX) * kSuper + within % kSuper);
  ty = static_cast<int>(static_cast<unsigned int>(st / supersX) * kSuper + within / kSuper);
  return static_cast<unsigned int>(tx) < p.tilesX && static_cast<unsigned int>(ty) < p.tilesY;
}

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
transposeTmaKernel(const __grid_constant__ CUtensorMap mapIn, const __grid_constant__ CUtensorMap mapOut, const __grid_constant__ TtParams p) {
  gridDependencyPrologue();
  extern __shared__ unsigned char smemRaw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  unsigned char *stages = smem;
  unsigned char *staging = smem + static_cast<size_t>(kStages) * kTileBytes;
  unsigned long long *full = reinterpret_cast<unsigned long long *>(staging + kWarps * kOutBuffers * kOutBytes);
  unsigned long long *empty = full + kStages;
  volatile int *abortFlag = reinterpret_cast<volatile int *>(empty + kStages);
  unsigned int *status = p.status ? p.status : &g_transposeStatus;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&full[s])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(&empty[s])), "r"(kWarps) : "memory");
    }
    *abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&mapIn) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&mapOut) : "memory");
  }
  __syncthreads();

  if (warp == kWarps) {
    // ---------------- producer ----------------
    if (lane == 0) {
      unsigned int it = 0;
      bool ok = true;
      for (unsigned long long t = blockIdx.x; t < p.numTiles && ok; t += gridDim.x) {
        int tx, ty;
        if (!tileOf(p, t, tx, ty)) continue;  // (the transposing warps skip the same tiles: `it` counts real ones)
        const unsigned int s = it % kStages, phase = (it / kStages) & 1u;
        ++it;
        if (!mbarWait(smemAddr(&empty[s]), phase ^ 1u, abortFlag, status)) { ok = false; break; }
        const unsigned int bar = smemAddr(&full[s]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kTileBytes) : "memory");
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                     ::"r"(smemAddr(stages + static_cast<size_t>(s) * kTileBytes)), "l"(&mapIn), "r"(tx * kTile), "r"(ty * kTile), "r"(bar)
                     : "memory");
      }
      if (!ok) {
        // loads already issued still land in this CTA's shared memory: give them time before the CTA ends
        for (int s = 0; s < kStages; ++s) {
          const unsigned long long t0 = globalTimerNs();
          while (!mbarTryWait(smemAddr(&full[s]), 0) && !mbarTryWait(smemAddr(&full[s]), 1) && globalTimerNs() - t0 < 1000000ull) {
          }
        }
      }
    }
    return;
  }

  // ---------------- transposing warps ----------------
  unsigned char *myStaging = staging + static_cast<size_t>(warp) * kOutBuffers * kOutBytes;
  unsigned int it = 0, buffer = 0;
  const int r8 = lane & 7, j = lane >> 3;
  for (unsigned long long t = blockIdx.x; t < p.numTiles; t += gridDim.x) {
    int tx, ty;
    if (!tileOf(p, t, tx, ty)) continue;
    const unsigned int s = it % kStages, phase = (it / kStages) & 1u;
    ++it;
    if (!mbarWait(smemAddr(&full[s]), phase, abortFlag, status)) break;
    // the store that last used this staging buffer must have read it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kOutBuffers - 1) : "memory");
    __syncwarp();
    const unsigned int src = smemAddr(stages + static_cast<size_t>(s) * kTileBytes);
    const unsigned int dst = smemAddr(myStaging + buffer * kOutBytes);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int cc = 2 * warp + (q >> 1);  // 16-byte column piece of the input tile = 8 output rows
      const int h = q & 1;                 // which half of the tile's 64 input rows (four 8-row blocks each)
      // four 8 x 8 blocks: input rows 8 (4h + j) .. + 7, columns 8 cc .. + 7; lane supplies row r8 of block j
      const unsigned int a = src + static_cast<unsigned int>((8 * (4 * h + j) + r8) * 128 + ((cc ^ r8) << 4));
      unsigned int v0, v1, v2, v3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(a) : "memory");
      // their transposes are rows 8 (q >> 1) .. + 7 of this warp's 16 output rows, 16-byte pieces 4h + j
      const int o = 8 * (q >> 1) + r8;
      const unsigned int d = dst + static_cast<unsigned int>(o * 128 + (((4 * h + j) ^ (o & 7)) << 4));
      asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(d), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copy engine must see what stmatrix wrote
    __syncwarp();
    if (lane == 0) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(&empty[s])) : "memory");  // this warp is done with the stage
      const int firstRow = tx * kTile + warp * kRowsPerWarp;
      if (firstRow < p.outRows)  // (a piece wholly below the output has nothing to write; one partly below is clipped)
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                     ::"l"(&mapOut), "r"(ty * kTile), "r"(firstRow), "r"(dst) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    buffer ^= 1u;
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all of this warp's stores are complete
  __syncwarp();
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

bool makeMap(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint64_t rowBytes, uint32_t boxInner, uint32_t boxOuter) {
  EncodeTiledFn fn = encodeTiled();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {rowBytes};
  cuuint32_t box[2] = {boxInner, boxOuter};
  cuuint32_t elemStrides[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A function attribute belongs to the function on the current device: set it once per device.
cudaError_t reserveSharedMemory() {
  static std::mutex mu;
  static bool done[64] = {false};
  int dev = 0;
  if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(transposeTmaKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
  if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
  return e;
}

} // namespace

bool transposeTmaApplies(const TransposeLaunch &l) {
  if (l.elemBytes != 2 || l.rows <= 0 || l.cols <= 0) return false;
  if (l.rows >= (1ll << 31) || l.cols >= (1ll << 31)) return false;
  const bool aligned = ((reinterpret_cast<uintptr_t>(l.in) | reinterpret_cast<uintptr_t>(l.out)) & 15u) == 0 &&
                       (l.inRowStride * 2) % 16 == 0 && (l.outRowStride * 2) % 16 == 0;
  // a tensor map's row pitch is below 2^40 bytes; rows shorter than a box would make every load mostly padding
  return aligned && l.inRowStride * 2 < (1ll << 40) && l.outRowStride * 2 < (1ll << 40) && l.inRowStride >= l.cols &&
         l.outRowStride >= l.rows && encodeTiled() != nullptr;
}

int launchTransposeTma(const TransposeLaunch &l, int smCount, cudaStream_t stream) {
  CUtensorMap mapIn, mapOut;
  if (!makeMap(&mapIn, l.in, static_cast<uint64_t>(l.cols), static_cast<uint64_t>(l.rows), static_cast<uint64_t>(l.inRowStride) * 2, kTile, kTile) ||
      !makeMap(&mapOut, l.out, static_cast<uint64_t>(l.rows), static_cast<uint64_t>(l.cols), static_cast<uint64_t>(l.outRowStride) * 2, kTile, kRowsPerWarp))
    return cudaErrorInvalidValue;
  if (const cudaError_t e = reserveSharedMemory(); e != cudaSuccess) return e;
  TtParams p = {};
  const long long tilesX = (l.cols + kTile - 1) / kTile, tilesY = (l.rows + kTile - 1) / kTile;
  p.tilesX = static_cast<unsigned int>(tilesX);
  p.tilesY = static_cast<unsigned int>(tilesY);
  // whole squares: the kernel skips the tiles of a border square that lie outside the matrix
  p.numTiles = static_cast<unsigned long long>((tilesX + kSuper - 1) / kSuper) * static_cast<unsigned long long>((tilesY + kSuper - 1) / kSuper) *
               (kSuper * kSuper);
  p.outRows = static_cast<int>(l.cols);
  p.status = l.status;
  const unsigned int grid = static_cast<unsigned int>(
      std::min<unsigned long long>(p.numTiles, static_cast<unsigned long long>(std::max(smCount, 1)) * kCtasPerSm));
  launchDependent(transposeTmaKernel, grid, kThreads, kSmemBytes, stream, mapIn, mapOut, p);
  return cudaGetLastError();
}

int transposeTmaCheckStatus(char *message, size_t messageBytes) {
  unsigned int word = 0;
  if (cudaMemcpyFromSymbol(&word, g_transposeStatus, sizeof(word)) != cudaSuccess || word == 0) return 0;
  const unsigned int zero = 0;
  cudaMemcpyToSymbol(g_transposeStatus, &zero, sizeof(zero));
  if (message && messageBytes) snprintf(message, messageBytes, "transpose: a wait for a staged tile ran out after 2 s");
  return 1;
}

} // namespace kernels
} // namespace afir
